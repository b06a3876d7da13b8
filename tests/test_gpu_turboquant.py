"""TurboQuant 8-bit KV: encoder bit-exact against the CPU oracle, decode attention within
tolerance (fp16 output, max abs error <= 2e-3 of the largest reference magnitude)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _c(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def dev():
    from ironmill_b200 import ops
    return ops.Device(0)


@pytest.fixture(scope="module")
def tqc():
    return orc.TqConstants(128, 8, seed=42)


@pytest.fixture(scope="module")
def tq(dev, tqc):
    from ironmill_b200 import ops
    return ops.TurboQuant(dev, 128, 8, tqc.signs, tqc.qjl, tqc.k_levels, tqc.k_bounds, tqc.v_levels, tqc.v_bounds)


def test_library_codebook_equals_oracle():
    from ironmill_b200 import ops
    for bits in (3, 4, 7, 8):
        lv, bd = ops.tq_lloyd_max(128, bits)
        rl, rb = orc.lloyd_max_gaussian(128, bits)
        assert (lv.view(np.uint32) == rl.view(np.uint32)).all() and (bd.view(np.uint32) == rb.view(np.uint32)).all()
    signs, qjl = ops.tq_generate(128, 42)
    assert set(np.unique(signs)) <= {-1.0, 1.0} and abs(float(qjl.mean())) < 0.05 and abs(float(qjl.std()) - 1) < 0.05


def _encode_both(tq, tqc, kv, is_k, nkv, max_seq, base, nseq=1):
    T = kv.size // (nseq * nkv * 128)
    cache = np.zeros((nseq, nkv, max_seq, 128), dtype=np.uint8)
    scale = np.zeros((nseq, nkv, max_seq), dtype=np.float32)
    rn = np.zeros((nseq, nkv, max_seq), dtype=np.float32)
    for s in range(nseq):
        orc.tq_encode(kv.reshape(nseq, T, nkv, 128)[s], tqc, is_k, cache[s], scale[s], rn[s], nkv, max_seq, base)
    cd, sd, rd = _c(np.zeros_like(cache)), _c(np.zeros_like(scale)), _c(np.zeros_like(rn))
    tq.encode(_c(kv), is_k, cd, sd, rd, nkv, max_seq, base, nseq=nseq)
    return (cache, scale, rn), (cd.cpu().numpy(), sd.cpu().numpy(), rd.cpu().numpy())


@pytest.mark.parametrize("is_k", [True, False])
@pytest.mark.parametrize("T,base,max_seq,nseq", [(1, 0, 64, 1), (5, 3, 64, 1), (33, 60, 64, 1), (2, 10, 32, 3)])
def test_encode_bit_exact(tq, tqc, is_k, T, base, max_seq, nseq):
    nkv = 8
    kv = H.make_x(nseq * T, nkv * 128, seed=T + base, name="kv")
    (c, s, r), (gc, gs, gr) = _encode_both(tq, tqc, kv, is_k, nkv, max_seq, base, nseq)
    assert (gc == c).all(), "cache bytes differ"
    assert (gs.view(np.uint32) == s.view(np.uint32)).all(), "scales differ"
    if is_k:
        assert (gr.view(np.uint32) == r.view(np.uint32)).all(), "residual norms differ"


def test_encode_edge_values(tq, tqc):
    kv = np.zeros((4, 8 * 128), dtype=np.float16)
    kv[1] = 1.0
    kv[2, ::7] = np.float16(65504.0)
    kv[3] = H.make_x(1, 8 * 128, 3)[0] * np.float16(1e-4)
    for is_k in (True, False):
        (c, s, r), (gc, gs, gr) = _encode_both(tq, tqc, kv, is_k, 8, 16, 0)
        assert (gc == c).all() and (gs.view(np.uint32) == s.view(np.uint32)).all() and (gr.view(np.uint32) == r.view(np.uint32)).all()


def _fill_cache(tq, tqc, nkv, max_seq, n, seed, nseq=1):
    k = H.make_x(nseq * n, nkv * 128, seed, "K")
    v = H.make_x(nseq * n, nkv * 128, seed, "V")
    kc, ks, kr = [_c(np.zeros(s, dtype=d)) for s, d in (((nseq, nkv, max_seq, 128), np.uint8), ((nseq, nkv, max_seq), np.float32), ((nseq, nkv, max_seq), np.float32))]
    vc, vs, vr = [_c(np.zeros(s, dtype=d)) for s, d in (((nseq, nkv, max_seq, 128), np.uint8), ((nseq, nkv, max_seq), np.float32), ((nseq, nkv, max_seq), np.float32))]
    tq.encode(_c(k), True, kc, ks, kr, nkv, max_seq, 0, nseq=nseq)
    tq.encode(_c(v), False, vc, vs, vr, nkv, max_seq, 0, nseq=nseq)
    return kc, ks, kr, vc, vs


@pytest.mark.parametrize("nh,nkv", [(32, 8), (16, 8), (8, 8)])
@pytest.mark.parametrize("ctx", [1, 31, 32, 33, 255, 256, 257, 1024])
def test_decode_attention(tq, tqc, nh, nkv, ctx):
    max_seq = 1100
    kc, ks, kr, vc, vs = _fill_cache(tq, tqc, nkv, max_seq, ctx, seed=ctx)
    q = H.make_x(1, nh * 128, seed=ctx, name="q")
    scale = 1.0 / np.sqrt(128.0)
    ref = orc.tq_attention(q, kc.cpu().numpy(), vc.cpu().numpy(), tqc, ks.cpu().numpy(), vs.cpu().numpy(), kr.cpu().numpy(),
                           scale, nh, nkv, max_seq, ctx - 1, num_splits=0)
    for splits in (0, 1, 3):
        out = tq.attention(_c(q), kc, vc, ks, vs, kr, scale, nh, nkv, max_seq, ctx - 1, num_splits=splits)
        assert H.rel_err(out.cpu().numpy().reshape(ref.shape), ref) <= 2e-3, f"splits={splits}"


def test_oracle_split_mode_equals_single_pass(tq, tqc):
    """The reference's split + reduce path against its single-pass path (CPU oracle both sides)."""
    nh, nkv, max_seq, ctx = 16, 8, 600, 513
    kc, ks, kr, vc, vs = [a.cpu().numpy() for a in _fill_cache(tq, tqc, nkv, max_seq, ctx, seed=9)]
    q = H.make_x(1, nh * 128, seed=1, name="q")
    a = orc.tq_attention(q, kc, vc, tqc, ks, vs, kr, 0.088, nh, nkv, max_seq, ctx - 1, num_splits=0)
    b = orc.tq_attention(q, kc, vc, tqc, ks, vs, kr, 0.088, nh, nkv, max_seq, ctx - 1, num_splits=5)
    assert H.rel_err(b, a) <= 2e-3


def test_prefill_attention_causal_and_batched(tq, tqc):
    """T > 1 (prefill over the quantized cache, causal length base+t+1) and nseq > 1."""
    nh, nkv, max_seq, base, T, nseq = 32, 8, 128, 20, 6, 2
    kc, ks, kr, vc, vs = _fill_cache(tq, tqc, nkv, max_seq, base + T, seed=5, nseq=nseq)
    q = H.make_x(nseq * T, nh * 128, seed=8, name="q")
    out = tq.attention(_c(q), kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, base, nseq=nseq).cpu().numpy()
    out = out.reshape(nseq, T, nh, 128)
    for s in range(nseq):
        ref = orc.tq_attention(q.reshape(nseq, T, -1)[s], kc[s].cpu().numpy(), vc[s].cpu().numpy(), tqc, ks[s].cpu().numpy(),
                               vs[s].cpu().numpy(), kr[s].cpu().numpy(), 0.0884, nh, nkv, max_seq, base)
        assert H.rel_err(out[s], ref) <= 2e-3


def test_attention_full_context_property(tq, tqc):
    """32k context (the oracle is not run): the output with every V row equal to one vector
    reproduces that vector's quantize-dequantize image, whatever the scores are."""
    nh, nkv, max_seq, ctx = 32, 8, 32768, 32768
    g = torch.Generator(device="cuda").manual_seed(1)
    k = torch.randn((ctx, nkv * 128), generator=g, device="cuda").half()
    v1 = torch.randn((1, nkv * 128), generator=g, device="cuda").half()
    v = v1.expand(ctx, -1).contiguous()
    kc = torch.zeros((1, nkv, max_seq, 128), dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    ks, kr, vs, vr = [torch.zeros((1, nkv, max_seq), dtype=torch.float32, device="cuda") for _ in range(4)]
    tq.encode(k, True, kc, ks, kr, nkv, max_seq, 0)
    tq.encode(v, False, vc, vs, vr, nkv, max_seq, 0)
    q = torch.randn((1, nh * 128), generator=g, device="cuda").half()
    out = tq.attention(q, kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, ctx - 1).float().reshape(nh, 128)
    # expected: dequantised V row 0 rotated back = signs-Hadamard of codebook[v bytes] * scale
    lv = torch.from_numpy(tqc.v_levels).cuda()
    for h in (0, 5, 31):
        kvh = h // (nh // nkv)
        vrot = lv[vc[0, kvh, 0].long()] * vs[0, kvh, 0]
        ref = torch.from_numpy(orc.hadamard_rotate(vrot.cpu().numpy(), tqc.signs)).cuda()
        assert float((out[h] - ref).abs().max()) <= 2e-3 * float(ref.abs().max()) + 1e-3


@pytest.mark.parametrize("ctx,nseq,nh,nkv", [(8192, 8, 32, 8), (1024, 32, 32, 8), (32768, 1, 4, 1), (131072, 1, 4, 1)])
def test_decode_attention_long_context_and_batches_against_the_oracle(tq, tqc, ctx, nseq, nh, nkv):
    """The attention benchmark's contexts and batches against the CPU oracle (single pass): 8k x batch 8 and 1k x batch 32
    with 32 query / 8 KV heads; 32k and 128k for one KV head's four query heads (the oracle is O(context) per head)."""
    max_seq = ctx
    kc, ks, kr, vc, vs = _fill_cache(tq, tqc, nkv, max_seq, ctx, seed=ctx % 1000 + nseq, nseq=nseq)
    q = H.make_x(nseq, nh * 128, seed=ctx % 977, name="q")
    scale = 1.0 / np.sqrt(128.0)
    out = tq.attention(_c(q), kc, vc, ks, vs, kr, scale, nh, nkv, max_seq, ctx - 1, nseq=nseq).cpu().numpy().reshape(nseq, nh, 128)
    kcn, vcn, ksn, vsn, krn = (a.cpu().numpy() for a in (kc, vc, ks, vs, kr))
    worst = 0.0
    for s in range(nseq):
        ref = orc.tq_attention(q[s:s + 1], kcn[s], vcn[s], tqc, ksn[s], vsn[s], krn[s], scale, nh, nkv, max_seq, ctx - 1, num_splits=0)
        worst = max(worst, H.rel_err(out[s], ref.reshape(nh, 128)))
    print(f"ctx {ctx} x {nseq} sequences: max error {worst:.2e} of the largest output")
    # the tensor-core kernel multiplies fp16 operands (f32 accumulation): 2e-3 up to 32k positions, measured 2.8e-3 at 128k
    assert worst <= (2e-3 if ctx <= 32768 else 4e-3), worst


def test_device_side_position_past_the_cache_is_clamped(tq, tqc):
    """Positions can live in device memory (decode graphs): a value the host never saw must not make the kernels read
    past a head's rows.  Position max_seq - 1 with two tokens: the second token's length is clamped to max_seq."""
    nh, nkv, max_seq = 8, 2, 64
    kc, ks, kr, vc, vs = _fill_cache(tq, tqc, nkv, max_seq, max_seq, seed=4)
    q = H.make_x(2, nh * 128, seed=2, name="q")
    pos = torch.tensor([max_seq - 1], dtype=torch.int32, device="cuda")
    out = tq.attention(_c(q), kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, 0, pos_dev=pos).cpu().numpy().reshape(2, nh, 128)
    ref = orc.tq_attention(q[0:1], kc[0].cpu().numpy(), vc[0].cpu().numpy(), tqc, ks[0].cpu().numpy(), vs[0].cpu().numpy(),
                           kr[0].cpu().numpy(), 0.0884, nh, nkv, max_seq, max_seq - 1, num_splits=0)
    # token 0 sees all max_seq positions; token 1 would see max_seq + 1 and is clamped to the same max_seq positions
    q1 = orc.tq_attention(q[1:2], kc[0].cpu().numpy(), vc[0].cpu().numpy(), tqc, ks[0].cpu().numpy(), vs[0].cpu().numpy(),
                          kr[0].cpu().numpy(), 0.0884, nh, nkv, max_seq, max_seq - 1, num_splits=0)
    assert H.rel_err(out[0], ref.reshape(nh, 128)) <= 2e-3
    assert np.isfinite(out).all() and H.rel_err(out[1], q1.reshape(nh, 128)) <= 2e-3


def test_sequence_overflow_is_reported(tq):
    from ironmill_b200 import CudaSysError
    z8 = torch.zeros((1, 8, 16, 128), dtype=torch.uint8, device="cuda")
    zf = torch.zeros((1, 8, 16), dtype=torch.float32, device="cuda")
    q = torch.zeros((1, 8 * 128), dtype=torch.float16, device="cuda")
    with pytest.raises(CudaSysError):
        tq.attention(q, z8, z8, zf, zf, zf, 1.0, 8, 8, 16, 16)


@pytest.mark.parametrize("with_norm", [True, False])
@pytest.mark.parametrize("T,base", [(1, 0), (1, 77), (5, 30)])
def test_fused_attention_block_equals_separate_kernels(tq, tqc, with_norm, T, base):
    """RoPE + cache write + query rotation in one launch: cache bytes and norms identical to the
    separate kernels (same fp16 K/V after RoPE), attention output within tolerance of the oracle path."""
    from ironmill_b200 import ops
    nh, nkv, hd, max_seq = 16, 8, 128, 128
    kc, ks, kr, vc, vs = _fill_cache(tq, tqc, nkv, max_seq, base, seed=3) if base else [
        _c(np.zeros(s, dtype=d)) for s, d in (((1, nkv, max_seq, 128), np.uint8), ((1, nkv, max_seq), np.float32),
                                              ((1, nkv, max_seq), np.float32), ((1, nkv, max_seq, 128), np.uint8),
                                              ((1, nkv, max_seq), np.float32))]
    qkv = H.make_x(T, (nh + 2 * nkv) * hd, seed=base + T, name="qkv")
    qw = (1.0 + 0.1 * H.rng_for("qw").standard_normal(hd)).astype(np.float16)
    kw = (1.0 + 0.1 * H.rng_for("kw").standard_normal(hd)).astype(np.float16)
    cos, sin = orc.rope_table(hd, max_seq, 1e6)
    # separate path on copies of the caches
    q = np.ascontiguousarray(qkv[:, :nh * hd]); k = np.ascontiguousarray(qkv[:, nh * hd:(nh + nkv) * hd]); v = np.ascontiguousarray(qkv[:, (nh + nkv) * hd:])
    qd, kd = _c(q), _c(k)
    if with_norm:
        ops.qk_norm_rope_(qd, kd, _c(qw), _c(kw), _c(cos), _c(sin), nh, nkv, hd, base, 1e-6)
    else:
        ops.rope_(qd, _c(cos), _c(sin), nh, hd, base)
        ops.rope_(kd, _c(cos), _c(sin), nkv, hd, base)
    kc2, ks2, kr2, vc2, vs2 = kc.clone(), ks.clone(), kr.clone(), vc.clone(), vs.clone()
    tq.encode(kd, True, kc2, ks2, kr2, nkv, max_seq, base)
    tq.encode(_c(v), False, vc2, vs2, torch.zeros_like(kr2), nkv, max_seq, base)
    ref = tq.attention(qd, kc2, vc2, ks2, vs2, kr2, 0.0884, nh, nkv, max_seq, base)
    out = ops.tq_fused_attention(tq, _c(qkv), nh, nkv, _c(cos), _c(sin), kc, vc, ks, vs, kr, 0.0884, max_seq, base,
                                 qw=_c(qw) if with_norm else None, kw=_c(kw) if with_norm else None)
    torch.cuda.synchronize()
    assert H.rel_err(out.cpu().numpy(), ref.cpu().numpy().reshape(out.shape)) <= 2e-3
    same = float((kc == kc2).float().mean())
    assert same >= 0.999, same   # a K value that differs in its last fp16 bit after RoPE can move a code
    assert torch.equal(vc, vc2) and torch.equal(vs, vs2)


# ---------------------------------------------------------------------------------------------- 4-bit cache (n_bits = 4)
@pytest.fixture(scope="module")
def tqc4():
    return orc.TqConstants(128, 4, seed=42)


@pytest.fixture(scope="module")
def tq4(dev, tqc4):
    from ironmill_b200 import ops
    return ops.TurboQuant(dev, 128, 4, tqc4.signs, tqc4.qjl, tqc4.k_levels, tqc4.k_bounds, tqc4.v_levels, tqc4.v_bounds)


def _encode4(tq4, tqc4, kv, is_k, nkv, max_seq, base):
    T = kv.size // (nkv * 128)
    cache = np.zeros((nkv, max_seq, 64), dtype=np.uint8)
    scale, rn = np.zeros((nkv, max_seq), np.float32), np.zeros((nkv, max_seq), np.float32)
    orc.tq_encode(kv.reshape(T, nkv, 128), tqc4, is_k, cache, scale, rn, nkv, max_seq, base)
    cd, sd, rd = _c(np.zeros((1, nkv, max_seq, 64), np.uint8)), _c(np.zeros((1, nkv, max_seq), np.float32)), _c(np.zeros((1, nkv, max_seq), np.float32))
    tq4.encode(_c(kv), is_k, cd, sd, rd, nkv, max_seq, base)
    return (cache, scale, rn), (cd.cpu().numpy()[0], sd.cpu().numpy()[0], rd.cpu().numpy()[0]), (cd, sd, rd)


@pytest.mark.parametrize("is_k", [True, False])
@pytest.mark.parametrize("T,base,max_seq", [(1, 0, 64), (5, 3, 64), (33, 60, 64)])
def test_encode_4bit_bit_exact(tq4, tqc4, is_k, T, base, max_seq):
    """3-bit index | QJL sign (K) or 4-bit index (V), two elements per byte, against the oracle: bytes and norms."""
    kv = H.make_x(T, 8 * 128, seed=T + base, name="kv4")
    (c, s, r), (gc, gs, gr), _ = _encode4(tq4, tqc4, kv, is_k, 8, max_seq, base)
    assert (gc == c).all(), "packed cache bytes differ"
    assert (gs.view(np.uint32) == s.view(np.uint32)).all()
    if is_k:
        assert (gr.view(np.uint32) == r.view(np.uint32)).all()


@pytest.mark.parametrize("nh,nkv", [(32, 8), (16, 8), (8, 8), (16, 2)])
@pytest.mark.parametrize("base,T", [(0, 16), (0, 100), (37, 50), (300, 257), (1000, 24)])
def test_prefill_flash_attention_against_the_oracle(tq, tqc, nh, nkv, base, T):
    """The prefill form (cached rows dequantised once, causal tensor-core pass: tq_prefill.cu) against the oracle's
    per-token turboquant_attention, and against the per-token CUDA kernel; 4, 2, 1 and 8 query heads per KV head."""
    max_seq = base + T + 5
    kc, ks, kr, vc, vs = _fill_cache(tq, tqc, nkv, max_seq, base + T, seed=base + T)
    q = H.make_x(T, nh * 128, seed=T, name="qp")
    ref = orc.tq_attention(q, kc[0].cpu().numpy(), vc[0].cpu().numpy(), tqc, ks[0].cpu().numpy(), vs[0].cpu().numpy(), kr[0].cpu().numpy(),
                           0.0884, nh, nkv, max_seq, base)
    out = tq.prefill_attention(_c(q), kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, base).cpu().numpy().reshape(ref.shape)
    tok = tq.attention(_c(q), kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, base).cpu().numpy().reshape(ref.shape)
    e_new, e_tok = H.rel_err(out, ref), H.rel_err(tok, ref)
    print(f"prefill attention nh {nh} nkv {nkv} base {base} T {T}: flash {e_new:.2e}, per-token kernel {e_tok:.2e}")
    assert e_new <= 2e-3, (e_new, e_tok)


@pytest.mark.parametrize("base,T", [(0, 40), (130, 70)])
def test_prefill_flash_attention_4bit(tq4, tqc4, base, T):
    nh, nkv = 16, 4
    max_seq = base + T + 3
    n = base + T
    k, v = H.make_x(n, nkv * 128, n, "K4p"), H.make_x(n, nkv * 128, n, "V4p")
    (kc, ks, kr), _, (kcd, ksd, krd) = _encode4(tq4, tqc4, k, True, nkv, max_seq, 0)
    (vc, vs, _r), _, (vcd, vsd, _rd) = _encode4(tq4, tqc4, v, False, nkv, max_seq, 0)
    q = H.make_x(T, nh * 128, seed=T, name="q4p")
    ref = orc.tq_attention(q, kc, vc, tqc4, ks, vs, kr, 0.0884, nh, nkv, max_seq, base)
    out = tq4.prefill_attention(_c(q), kcd, vcd, ksd, vsd, krd, 0.0884, nh, nkv, max_seq, base).cpu().numpy().reshape(ref.shape)
    assert H.rel_err(out, ref) <= 2e-3


@pytest.mark.parametrize("nh,nkv", [(32, 8), (16, 8), (8, 8), (16, 2)])
@pytest.mark.parametrize("ctx", [1, 33, 257, 1024, 4097])
def test_decode_attention_4bit(tq4, tqc4, nh, nkv, ctx):
    """nh / nkv = 8 takes the f32 kernel (nibbles spread to bytes in shared memory), the others the tensor-core kernel."""
    max_seq = ctx + 3
    k, v = H.make_x(ctx, nkv * 128, ctx, "K4"), H.make_x(ctx, nkv * 128, ctx, "V4")
    (kc, ks, kr), _, (kcd, ksd, krd) = _encode4(tq4, tqc4, k, True, nkv, max_seq, 0)
    (vc, vs, _r), _, (vcd, vsd, _rd) = _encode4(tq4, tqc4, v, False, nkv, max_seq, 0)
    q = H.make_x(1, nh * 128, seed=ctx, name="q4")
    scale = 1.0 / np.sqrt(128.0)
    ref = orc.tq_attention(q, kc, vc, tqc4, ks, vs, kr, scale, nh, nkv, max_seq, ctx - 1, num_splits=0)
    for splits in (0, 3):
        out = tq4.attention(_c(q), kcd, vcd, ksd, vsd, krd, scale, nh, nkv, max_seq, ctx - 1, num_splits=splits)
        assert H.rel_err(out.cpu().numpy().reshape(ref.shape), ref) <= 2e-3, f"splits={splits}"
