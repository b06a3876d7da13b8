"""Pins the CPU oracle to the known-answer vectors of the reference's own unit tests.

Each test names the reference test it replays (paths relative to the reference root):
crates/mil-rs/src/ir/passes/affine_quantize.rs, int4_pack.rs,
crates/ironmill-core/src/dequant.rs, crates/ironmill-core/src/rope.rs,
crates/ironmill-inference/src/turboquant/codebook.rs.
"""
import numpy as np

from oracle import oracle as orc

EPS = float(np.finfo(np.float32).eps)


# --- affine_quantize.rs -------------------------------------------------------
def test_int4_per_tensor_known_values():
    # affine_quantize.rs:585-598
    q, s, zp = orc.quantize_affine([-3.0, 0.0, 3.0, 6.0, 12.0], 15.0)
    assert abs(s - 1.0) < 1e-6 and abs(zp - 3.0) < 1e-6
    assert q.tolist() == [0, 3, 6, 9, 15]


def test_int4_per_tensor_basic():
    # affine_quantize.rs:551-581: [0,1,2,3] -> scale 0.2, zp 0, ends map to 0 and 15
    q, s, zp = orc.quantize_affine([0.0, 1.0, 2.0, 3.0], 15.0)
    assert q[0] == 0 and q[3] == 15 and (q <= 15).all()
    assert abs(s - 0.2) < 1e-6 and zp == 0.0


def test_round_trips():
    # affine_quantize.rs:600-615 (int4), 873-890 (int8), 617-628 (negative range)
    for vals, qmax in (([-2.0, -0.5, 0.0, 1.5, 3.0], 15.0),
                       ([-3.0, -1.5, 0.0, 1.5, 3.0, 6.0], 255.0),
                       ([-10.0, -8.0, -5.0, -1.0], 15.0)):
        q, s, zp = orc.quantize_affine(vals, qmax)
        rec = orc.dequantize_affine_f32(q, s, zp)
        tol = s / 2.0 + EPS
        assert np.all(np.abs(np.asarray(vals, dtype=np.float32) - rec) <= tol)
    q, _, _ = orc.quantize_affine([-10.0, -8.0, -5.0, -1.0], 15.0)
    assert q[0] == 0 and q[3] == 15


def test_per_group_scales():
    # affine_quantize.rs:723-762: scales [1.0, 1/15]
    w = np.array([[0, 0, 0, 15, 0, 0, 0, 1]], dtype=np.float32)
    codes, scales, zps = orc.quantize_groups(w, 4, 4)
    assert scales.shape == (1, 2)
    assert abs(scales[0, 0] - 1.0) < 1e-5 and abs(scales[0, 1] - 1.0 / 15.0) < 1e-5


def test_per_group_basic_shapes():
    # affine_quantize.rs:633-720: [2,8], gs 4 -> scale/zp [2,2], wide group has larger scale
    w = np.array([[0, 1, 2, 3, 4, 5, 6, 7], [-1, 0, 1, 2, 10, 20, 30, 40]], dtype=np.float32)
    codes, scales, zps = orc.quantize_groups(w, 4, 4)
    assert codes.shape == (2, 8) and scales.shape == (2, 2) and zps.shape == (2, 2)
    assert (codes <= 15).all() and (scales > 0).all() and scales[1, 1] > scales[0, 0]
    assert orc.pack_int4(codes).size == 8


def test_partial_last_group():
    # affine_quantize.rs:765-796: [1,6] gs 4 -> two groups, 3 packed bytes
    w = np.array([[0, 1, 2, 3, 10, 20]], dtype=np.float32)
    codes, scales, zps = orc.quantize_groups(w, 4, 4)
    assert scales.shape == (1, 2)
    assert orc.pack_int4(codes).size == 3


def test_group_larger_than_tensor_and_equal_dim():
    # affine_quantize.rs:952-1004
    codes, scales, _ = orc.quantize_groups(np.array([[1, 2, 3, 4]], dtype=np.float32), 128, 4)
    assert scales.shape == (1, 1) and orc.pack_int4(codes).size == 2
    _, scales, _ = orc.quantize_groups(np.arange(8, dtype=np.float32).reshape(2, 4), 4, 4)
    assert scales.shape == (2, 1)


def test_uniform_and_single_and_empty():
    # affine_quantize.rs:893-949 (uniform weights, single weight), 1118-1123 (empty slice)
    for qmax in (15.0, 255.0):
        q, s, zp = orc.quantize_affine([42.0] * 8, qmax)
        assert len(set(q.tolist())) == 1 and q[0] <= qmax and s == 1.0
    q, s, zp = orc.quantize_affine([7.5], 15.0)
    assert q.size == 1 and q[0] <= 15
    q, s, zp = orc.quantize_affine([], 15.0)
    assert q.size == 0 and s == 1.0 and zp == 0.0


def test_non_finite_inputs():
    # affine_quantize.rs:262-277: non-finite values are skipped for min/max; none finite -> zeros
    q, s, zp = orc.quantize_affine([np.inf, np.nan, -np.inf], 15.0)
    assert q.tolist() == [0, 0, 0] and s == 1.0 and zp == 0.0
    q, s, zp = orc.quantize_affine([0.0, np.nan, 15.0, np.inf, -np.inf], 15.0)
    assert s == 1.0 and zp == 0.0 and q.tolist() == [0, 0, 15, 15, 0]


def test_int8_per_group_same_routine():
    # affine_quantize.rs:821-870: the 8-bit path is the same routine with qmax 255
    rng = np.random.default_rng(0)
    w = rng.standard_normal((4, 64)).astype(np.float32)
    codes, scales, zps = orc.quantize_groups(w, 64, 8)
    for r in range(4):
        q, s, zp = orc.quantize_affine(w[r], 255.0)
        assert (q == codes[r]).all() and s == scales[r, 0] and zp == zps[r, 0]


def test_quantize_matches_numpy_restatement():
    """The C routine against an independent numpy restatement of the same formula
    (f32 division, round half away from zero, clamp)."""
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((16, 512)) * 0.02).astype(np.float16)
    codes, scales, zps = orc.quantize_groups(w, 128, 4)
    wf = w.astype(np.float32).reshape(16, 4, 128)
    mn, mx = wf.min(-1), wf.max(-1)
    s = ((mx - mn) / np.float32(15.0)).astype(np.float32)
    t = (-mn / s).astype(np.float32)
    zp = np.copysign(np.floor(np.abs(t) + np.float32(0.5)), t).astype(np.float32)
    v = (wf / s[..., None] + zp[..., None]).astype(np.float32)
    q = np.clip(np.copysign(np.floor(np.abs(v) + np.float32(0.5)), v), 0, 15).astype(np.uint8)
    assert (s == scales).all() and (zp == zps).all()
    assert (q.reshape(16, 512) == codes).all()


# --- int4_pack.rs ---------------------------------------------------------------
def test_pack_vectors():
    # int4_pack.rs:100-146
    v = list(range(16))
    assert orc.unpack_int4(orc.pack_int4(v), 16).tolist() == v
    assert orc.pack_int4([3, 12]).tolist() == [0xC3]
    assert orc.pack_int4([5]).tolist() == [0x05] and orc.unpack_int4([0x05], 1).tolist() == [5]
    assert orc.unpack_int4(orc.pack_int4([1, 2, 3, 4]), 3).tolist() == [1, 2, 3]
    assert orc.pack_int4([]).size == 0
    assert orc.pack_int4([0xFF, 0xFF]).tolist() == [0xFF]
    assert orc.unpack_int4([0xFF], 2).tolist() == [15, 15]


def test_pack_u32_word_view():
    # int4_pack.rs:160-170: eight values 0..7 read as a little-endian u32 give 0x76543210
    packed = orc.pack_int4(list(range(8)))
    assert packed.view("<u4")[0] == 0x76543210
    vals = [3, 14, 1, 5, 9, 0, 15, 7, 2, 11]   # :222-231 cross-format consistency
    assert orc.unpack_int4(orc.pack_int4(vals), len(vals)).tolist() == vals


# --- ironmill-core dequant.rs --------------------------------------------------
def test_dequant_per_tensor_int8():
    # dequant.rs:404-430
    out = orc.dequant_affine([0, 1, 128, 255], np.float32([0.5]), np.float32([0.0]), (2, 2), 8)
    o = out.astype(np.float32).reshape(-1)
    assert abs(o[0]) < 1e-3 and abs(o[1] - 0.5) < 1e-3 and abs(o[2] - 64.0) < 1e-1 and abs(o[3] - 127.5) < 1.0


def test_dequant_per_axis_fp16_params():
    # dequant.rs:432-463
    out = orc.dequant_affine([10, 20, 30, 5, 10, 15], np.float16([0.1, 0.5]), np.float16([10.0, 5.0]),
                             (2, 3), 8, axis=0).astype(np.float32).reshape(-1)
    exp = [0.0, 1.0, 2.0, 0.0, 2.5, 5.0]
    for a, e, tol in zip(out, exp, [1e-2, 1e-2, 1e-2, 1e-2, 1e-1, 1e-1]):
        assert abs(a - e) < tol


def test_dequant_per_group_int4_low_nibble_first():
    # dequant.rs:102-139: (q - z) * s, low nibble first, group = col / gs
    codes = np.array([[1, 2, 3, 4, 5, 6, 7, 8]], dtype=np.uint8)
    packed = orc.pack_int4(codes)
    s = np.float32([[0.5, 2.0]])
    z = np.float32([[1.0, 4.0]])
    out = orc.dequant_affine(packed, s, z, (1, 8), 4, group_size=4).astype(np.float32)
    assert out.reshape(-1).tolist() == [0.0, 0.5, 1.0, 1.5, 2.0, 4.0, 6.0, 8.0]


def test_params_to_f16_rne():
    # dequant.rs:305-345: f32 -> f16 round to nearest even
    a = np.float32([1.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8, -0.1])
    assert (orc.f32_to_f16(a) == a.astype(np.float16)).all()


# --- rope.rs ---------------------------------------------------------------------
def test_rope_table():
    # rope.rs:55-75
    cos, sin = orc.rope_table(4, 2, 10000.0)
    assert cos.shape == (2, 2) and cos[0, 0] == np.float16(1.0) and sin[0, 0] == np.float16(0.0)
    cos, sin = orc.rope_table(8, 1, 10000.0, rotary_dim=4)
    assert (cos[0, 2:] == np.float16(1.0)).all() and (sin[0, 2:] == np.float16(0.0)).all()
    cos, sin = orc.rope_table(128, 64, 1e6)
    i = np.arange(64, dtype=np.float64)
    freq = 1.0 / np.power(1e6, 2.0 * i / 128.0)
    ang = np.arange(64, dtype=np.float64)[:, None] * freq[None, :]
    # libm cos/sin may differ from numpy in the last ulp of f64; after f16 rounding they agree
    assert (cos == np.cos(ang).astype(np.float16)).mean() > 0.999
    assert (sin == np.sin(ang).astype(np.float16)).mean() > 0.999


# --- codebook.rs -------------------------------------------------------------------
def test_codebook_properties():
    # codebook.rs:206-255: sorted, symmetric, scales with dim, 8 levels at 3 bits
    for dim in (64, 128, 256):
        lv, bd = orc.lloyd_max_gaussian(dim, 4)
        assert lv.size == 16 and bd.size == 15
        assert (np.diff(lv) > 0).all() and (np.diff(bd) > 0).all()
        assert np.abs(lv[:8] + lv[::-1][:8]).max() < 1e-5
    m = [orc.lloyd_max_gaussian(d, 4)[0][-1] for d in (64, 128, 256)]
    assert m[0] > m[1] > m[2]
    lv, bd = orc.lloyd_max_gaussian(128, 3)
    assert lv.size == 8 and bd.size == 7


def test_codebook_is_lloyd_max_fixed_point():
    """The published optimality conditions: boundaries are midpoints and each level is the
    conditional mean of N(0, 1/d) over its cell (checked by numerical integration)."""
    for bits in (7, 8):
        lv, bd = orc.lloyd_max_gaussian(128, bits)
        assert lv.size == 1 << bits
        assert np.allclose(bd, (lv[:-1].astype(np.float64) + lv[1:]) / 2, atol=1e-7)
        sigma = 1 / np.sqrt(128.0)
        edges = np.concatenate([[-8 * sigma], bd.astype(np.float64), [8 * sigma]])
        for i in (0, 1, (1 << bits) // 2, (1 << bits) - 2, (1 << bits) - 1):
            xs = np.linspace(edges[i], edges[i + 1], 20001)
            pdf = np.exp(-0.5 * (xs / sigma) ** 2)
            mean = (xs * pdf).sum() / pdf.sum()
            # the reference's erf approximation is good to ~1.5e-7 absolute, which is ~1e-3
            # relative to the probability mass of a tail cell: tail cells are the loosest
            assert abs(mean - lv[i]) < 5e-3 * sigma


def test_codebook_tables_are_not_monotone_at_7_and_8_bits():
    """Restated behaviour, kept on purpose: the tail branch of the reference's inverse-normal
    approximation (codebook.rs:150-184) returns values near zero for p < 0.08, so the 20 outermost
    initial levels per side of a 128- or 256-level table start out of order and the Lloyd iterations
    never untangle them.  The encoder's linear scan (last boundary <= u) is what defines the
    index, and both the oracle and the CUDA encoder reproduce exactly that."""
    for bits in (7, 8):
        lv, bd = orc.lloyd_max_gaussian(128, bits)
        assert (np.diff(bd) <= 0).any()
        assert np.abs(lv + lv[::-1]).max() < 1e-5   # still symmetric


def test_argmax_last_max_wins():
    # crates/ironmill-inference/src/sampling.rs:331-339: max_by keeps the last of equal maxima
    assert orc.argmax([1.0, 3.0, 3.0, 2.0]) == 2
    assert orc.argmax([5.0]) == 0
