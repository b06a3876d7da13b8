"""numpy front end of the CPU oracle (oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product package never imports it.

Arrays are numpy; fp16 tensors are passed as ``np.float16`` and viewed as
uint16 at the C boundary.  Each wrapper names the C function it calls; the
reference file:line each one follows is cited in oracle.c.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile oracle.c with the Makefile beside it (gcc, -ffp-contract=off)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_argmax.restype = C.c_uint32
        _lib.orc_max_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _h(a):
    """Contiguous fp16 array (or None)."""
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def _f(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float32, a.dtype
    return a


def _u8(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8, a.dtype
    return a


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---------------------------------------------------------------- quantize / pack
def quantize_affine(values, qmax: float):
    """orc_quantize_affine -> (codes u8, scale, zero_point)."""
    v = _f(np.asarray(values, dtype=np.float32))
    q = np.zeros(v.size, dtype=np.uint8)
    s = C.c_float()
    z = C.c_float()
    lib().orc_quantize_affine(_p(v), C.c_size_t(v.size), C.c_float(qmax), _p(q), C.byref(s), C.byref(z))
    return q, float(np.float32(s.value)), float(np.float32(z.value))


def dequantize_affine_f32(q, scale: float, zp: float):
    q = _u8(np.asarray(q, dtype=np.uint8))
    out = np.zeros(q.size, dtype=np.float32)
    lib().orc_dequantize_affine_f32(_p(q), C.c_size_t(q.size), C.c_float(scale), C.c_float(zp), _p(out))
    return out


def quantize_groups(w, group_size: int, bits: int, awq=None, threads: int = 1):
    """Per-group affine quantization of a [rows, K] tensor (fp16 or f32 input).

    Returns (codes u8 [rows,K], scales f32 [rows,G], zero_points f32 [rows,G])."""
    w = np.ascontiguousarray(w)
    rows = int(np.prod(w.shape[:-1])) if w.ndim > 1 else 1
    K = w.shape[-1]
    G = -(-K // group_size)
    codes = np.zeros((rows, K), dtype=np.uint8)
    scales = np.zeros((rows, G), dtype=np.float32)
    zps = np.zeros((rows, G), dtype=np.float32)
    if w.dtype == np.float16:
        lib().orc_quantize_groups_f16(_p(w), C.c_size_t(rows), C.c_size_t(K), C.c_size_t(group_size),
                                      C.c_int(bits), _p(_h(awq)), _p(codes), _p(scales), _p(zps),
                                      C.c_int(threads))
    else:
        assert awq is None
        w = _f(w.astype(np.float32, copy=False))
        lib().orc_quantize_groups_f32(_p(w), C.c_size_t(rows), C.c_size_t(K), C.c_size_t(group_size),
                                      C.c_int(bits), _p(codes), _p(scales), _p(zps))
    return codes, scales, zps


def pack_int4(values):
    v = _u8(np.asarray(values, dtype=np.uint8).reshape(-1))
    out = np.zeros((v.size + 1) // 2, dtype=np.uint8)
    lib().orc_pack_int4(_p(v), C.c_size_t(v.size), _p(out))
    return out


def unpack_int4(packed, count: int):
    p = _u8(np.asarray(packed, dtype=np.uint8).reshape(-1))
    out = np.zeros(count, dtype=np.uint8)
    lib().orc_unpack_int4(_p(p), C.c_size_t(count), _p(out))
    return out


def f32_to_f16(a):
    a = _f(np.asarray(a, dtype=np.float32))
    out = np.zeros(a.shape, dtype=np.float16)
    lib().orc_f32_to_f16(_p(a), C.c_size_t(a.size), _p(out))
    return out


def dequant_affine(qdata, scale, zp, shape, bits: int, group_size=None, axis=None):
    """orc_dequant_affine: fp16 tensor f16((q - z) * s); scale/zp f32 or fp16 arrays."""
    qdata = _u8(np.asarray(qdata, dtype=np.uint8).reshape(-1))
    scale = np.ascontiguousarray(scale)
    zp = np.ascontiguousarray(zp)
    total = int(np.prod(shape))
    out = np.zeros(total, dtype=np.float16)
    K = shape[-1] if len(shape) else 1
    if group_size is not None:
        mode, axis_size, stride, gs = 0, 0, 0, group_size
    elif axis is not None:
        mode, gs = 1, 0
        axis_size = shape[axis]
        stride = int(np.prod(shape[axis + 1:])) if axis + 1 < len(shape) else 1
    else:
        mode, axis_size, stride, gs = 2, 0, 0, 0
    lib().orc_dequant_affine(_p(qdata), _p(scale), _p(zp), C.c_int(scale.dtype == np.float32),
                             C.c_int(zp.dtype == np.float32), C.c_int(mode), C.c_size_t(total),
                             C.c_size_t(K), C.c_size_t(gs), C.c_size_t(axis_size), C.c_size_t(stride),
                             C.c_int(bits), _p(out))
    return out.reshape(shape)


# ---------------------------------------------------------------- matvec family
def matvec_affine(qdata, scales_f16, zeros_f16, x, N, K, group_size, bits, awq=None, threads=1):
    x = _h(x).reshape(-1, K)
    B = x.shape[0]
    y = np.zeros((B, N), dtype=np.float16)
    lib().orc_matvec_affine(_p(_u8(qdata)), _p(_h(scales_f16)), _p(_h(zeros_f16)), _p(_h(awq)), _p(x), _p(y),
                            C.c_size_t(N), C.c_size_t(K), C.c_size_t(group_size), C.c_int(bits),
                            C.c_size_t(B), C.c_int(threads))
    return y


def matmul_affine(qdata, scales_f16, zeros_f16, a, N, K, group_size, bits, awq=None, threads=1):
    a = _h(a).reshape(-1, K)
    M = a.shape[0]
    c = np.zeros((M, N), dtype=np.float16)
    lib().orc_matmul_affine(_p(_u8(qdata)), _p(_h(scales_f16)), _p(_h(zeros_f16)), _p(_h(awq)), _p(a), _p(c),
                            C.c_size_t(M), C.c_size_t(N), C.c_size_t(K), C.c_size_t(group_size),
                            C.c_int(bits), C.c_int(threads))
    return c


def ffn_gate_up_act(gq, gs, gz, uq, us, uz, x, I, K, group_size, bits, awq=None, threads=1):
    x = _h(x).reshape(-1, K)
    B = x.shape[0]
    out = np.zeros((B, I), dtype=np.float16)
    lib().orc_ffn_gate_up_act(_p(_u8(gq)), _p(_h(gs)), _p(_h(gz)), _p(_u8(uq)), _p(_h(us)), _p(_h(uz)),
                              _p(_h(awq)), _p(x), _p(out), C.c_size_t(I), C.c_size_t(K),
                              C.c_size_t(group_size), C.c_int(bits), C.c_size_t(B), C.c_int(threads))
    return out


def fused_residual_norm_matvec(a, b, gamma, qdata, scales_f16, zeros_f16, eps, N, K, group_size, bits,
                               awq=None, threads=1):
    a = _h(a).reshape(-1, K)
    b = _h(b).reshape(-1, K)
    B = a.shape[0]
    y = np.zeros((B, N), dtype=np.float16)
    res = np.zeros((B, K), dtype=np.float16)
    nrm = np.zeros((B, K), dtype=np.float16)
    lib().orc_fused_residual_norm_matvec(_p(a), _p(b), _p(_h(gamma)), _p(_u8(qdata)), _p(_h(scales_f16)),
                                         _p(_h(zeros_f16)), _p(_h(awq)), C.c_float(eps), _p(y), _p(res), _p(nrm),
                                         C.c_size_t(N), C.c_size_t(K), C.c_size_t(group_size), C.c_int(bits),
                                         C.c_size_t(B), C.c_int(threads))
    return y, res, nrm


def matvec_f16(w, x, threads=1):
    w = _h(w)
    N, K = w.shape
    x = _h(x).reshape(-1, K)
    B = x.shape[0]
    y = np.zeros((B, N), dtype=np.float16)
    lib().orc_matvec_f16(_p(w), _p(x), _p(y), C.c_size_t(N), C.c_size_t(K), C.c_size_t(B), C.c_int(threads))
    return y


# ---------------------------------------------------------------- norms / embedding / rope
def rms_norm(x, gamma, eps):
    x = _h(x)
    H = x.shape[-1]
    T = x.size // H
    out = np.zeros_like(x)
    lib().orc_rms_norm(_p(x), _p(_h(gamma)), _p(out), C.c_size_t(H), C.c_size_t(T), C.c_float(eps))
    return out


def fused_residual_rms_norm(a, b, gamma, eps):
    a = _h(a)
    b = _h(b)
    H = a.shape[-1]
    T = a.size // H
    normed = np.zeros_like(a)
    residual = np.zeros_like(a)
    lib().orc_fused_residual_rms_norm(_p(a), _p(b), _p(_h(gamma)), _p(normed), _p(residual),
                                      C.c_size_t(H), C.c_size_t(T), C.c_float(eps))
    return normed, residual


def residual_add(a, b):
    a = _h(a)
    b = _h(b)
    out = np.zeros_like(a)
    lib().orc_residual_add(_p(a), _p(b), _p(out), C.c_size_t(a.size))
    return out


def embedding_norm(tokens, table, gamma, eps, embed_scale=1.0):
    tokens = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint32))
    table = _h(table)
    vocab, H = table.shape
    T = tokens.size
    normed = np.zeros((T, H), dtype=np.float16)
    raw = np.zeros((T, H), dtype=np.float16)
    lib().orc_embedding_norm(_p(tokens), _p(table), _p(_h(gamma)), _p(normed), _p(raw), C.c_size_t(H),
                             C.c_size_t(T), C.c_size_t(vocab), C.c_float(eps), C.c_float(embed_scale))
    return normed, raw


def rope_table(head_dim, max_pos, theta, rotary_dim=None):
    half = head_dim // 2
    cos = np.zeros((max_pos, half), dtype=np.float16)
    sin = np.zeros((max_pos, half), dtype=np.float16)
    lib().orc_rope_table(C.c_size_t(head_dim), C.c_size_t(max_pos), C.c_double(theta),
                         C.c_size_t(rotary_dim or 0), _p(cos), _p(sin))
    return cos, sin


def rope(qk, cos, sin, heads, hd, seq_offset):
    """In place on a copy; qk [T, heads, hd] fp16."""
    qk = _h(qk).copy()
    T = qk.size // (heads * hd)
    lib().orc_rope(_p(qk), _p(_h(cos)), _p(_h(sin)), C.c_size_t(heads), C.c_size_t(hd),
                   C.c_size_t(seq_offset), C.c_size_t(T))
    return qk


def qk_norm_rope(q, k, qw, kw, cos, sin, nh, nkv, hd, seq_offset, eps, rotary_dim=None):
    q = _h(q).copy()
    k = _h(k).copy()
    T = q.size // (nh * hd)
    lib().orc_qk_norm_rope(_p(q), _p(k), _p(_h(qw)), _p(_h(kw)), _p(_h(cos)), _p(_h(sin)), C.c_size_t(nh),
                           C.c_size_t(nkv), C.c_size_t(hd), C.c_size_t(rotary_dim or hd),
                           C.c_size_t(seq_offset), C.c_size_t(T), C.c_float(eps))
    return q, k


# ---------------------------------------------------------------- TurboQuant
def lloyd_max_gaussian(dim, n_bits):
    n = 1 << n_bits
    levels = np.zeros(n, dtype=np.float32)
    bounds = np.zeros(n - 1, dtype=np.float32)
    lib().orc_lloyd_max_gaussian(C.c_size_t(dim), C.c_int(n_bits), _p(levels), _p(bounds))
    return levels, bounds


def hadamard_rotate(x, signs):
    x = _f(np.asarray(x, dtype=np.float32)).copy()
    lib().orc_hadamard_rotate(_p(x), _p(_f(signs)), C.c_size_t(x.size))
    return x


class TqConstants:
    """Rotation signs, QJL matrix and K/V codebooks for one head_dim / n_bits.

    Codebooks follow the reference's Lloyd-Max routine.  The reference draws signs and the
    QJL matrix from the `rand` crate's StdRng (unpinned); here a seeded numpy generator
    provides a valid +-1 vector and an N(0,1) matrix, and both sides of every comparison
    are handed these same arrays."""

    def __init__(self, head_dim=128, n_bits=8, seed=42):
        rng = np.random.Generator(np.random.PCG64(seed))
        self.head_dim = head_dim
        self.n_bits = n_bits
        self.signs = np.where(rng.random(head_dim) < 0.5, 1.0, -1.0).astype(np.float32)
        rng2 = np.random.Generator(np.random.PCG64(seed + 1))
        self.qjl = rng2.standard_normal((head_dim, head_dim)).astype(np.float32)
        self.k_levels, self.k_bounds = lloyd_max_gaussian(head_dim, n_bits - 1)
        self.v_levels, self.v_bounds = lloyd_max_gaussian(head_dim, n_bits)


def tq_encode(kv, tq: TqConstants, is_k, cache, scale_buf, r_norms, nkv, max_seq, base_pos):
    """orc_tq_encode; writes into cache / scale_buf / r_norms in place. kv [T, nkv, hd] fp16."""
    kv = _h(kv)
    hd = tq.head_dim
    T = kv.size // (nkv * hd)
    cb, bd = (tq.k_levels, tq.k_bounds) if is_k else (tq.v_levels, tq.v_bounds)
    assert cache.dtype == np.uint8 and cache.flags.c_contiguous
    lib().orc_tq_encode(_p(kv), _p(tq.signs), _p(cb), _p(bd), _p(tq.qjl), C.c_int(int(is_k)),
                        C.c_int(tq.n_bits), _p(cache), _p(scale_buf), _p(r_norms if r_norms is not None else scale_buf),
                        C.c_size_t(nkv), C.c_size_t(hd), C.c_size_t(max_seq), C.c_size_t(base_pos), C.c_size_t(T))


def tq_attention(q, k_cache, v_cache, tq: TqConstants, k_scale, v_scale, k_rnorm, attn_scale, nh, nkv,
                 max_seq, base_pos, num_splits=0):
    q = _h(q)
    hd = tq.head_dim
    T = q.size // (nh * hd)
    out = np.zeros((T, nh, hd), dtype=np.float16)
    lib().orc_tq_attention(_p(q), _p(_u8(k_cache)), _p(_u8(v_cache)), _p(tq.signs), _p(_f(k_scale)),
                           _p(_f(v_scale)), _p(tq.k_levels), _p(tq.v_levels), _p(tq.qjl), _p(_f(k_rnorm)),
                           C.c_float(attn_scale), C.c_int(tq.n_bits), _p(out), C.c_size_t(nh), C.c_size_t(nkv),
                           C.c_size_t(hd), C.c_size_t(max_seq), C.c_size_t(base_pos), C.c_size_t(T),
                           C.c_size_t(num_splits))
    return out


def sdpa_f16(q, k_cache, v_cache, scale, nh, nkv, hd, max_seq, base_pos, num_splits=0):
    """fp16-KV attention (fused_sdpa / prefill_attention_v2; num_splits > 0: fused_sdpa_split + fused_sdpa_reduce).
    q [T, nh, hd], caches [nkv, max_seq, hd] fp16 -> [T, nh, hd] fp16."""
    q = _h(q)
    T = q.size // (nh * hd)
    out = np.zeros((T, nh, hd), dtype=np.float16)
    lib().orc_sdpa_f16(_p(q), _p(_h(k_cache)), _p(_h(v_cache)), C.c_float(scale), _p(out), C.c_size_t(nh), C.c_size_t(nkv),
                       C.c_size_t(hd), C.c_size_t(max_seq), C.c_size_t(base_pos), C.c_size_t(T), C.c_size_t(num_splits))
    return out


def argmax(logits):
    logits = _f(np.asarray(logits, dtype=np.float32))
    return int(lib().orc_argmax(_p(logits), C.c_size_t(logits.size)))
