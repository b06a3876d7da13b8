"""Kernel-level entry points of the C ABI, called with torch CUDA tensors.

torch supplies device memory and streams only; every computation below is a call into
libironmill_cuda.so.  Names follow the reference's kernels
(crates/ironmill-inference/src/metal/shaders/**) and quantizer
(crates/mil-rs/src/ir/passes/affine_quantize.rs).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ._lib import IM_DTYPE_F16, IM_DTYPE_F32, check, lib, vp


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Device:
    """MetalDevice counterpart (crates/ironmill-metal-sys/src/device.rs:74-260)."""

    def __init__(self, ordinal: int = 0):
        self.handle = C.c_void_p()
        check(lib().im_cuda_device_open(C.c_int(ordinal), C.byref(self.handle)))
        self.ordinal = ordinal

    @property
    def name(self) -> str:
        buf = C.create_string_buffer(256)
        check(lib().im_cuda_device_name(self.handle, buf, C.c_size_t(256)))
        return buf.value.decode()

    @property
    def sm_count(self) -> int:
        return int(lib().im_cuda_device_sm_count(self.handle))

    def allocated_bytes(self) -> int:
        return int(lib().im_cuda_device_allocated_bytes(self.handle))

    def synchronize(self) -> None:
        check(lib().im_cuda_device_synchronize(self.handle))

    def close(self) -> None:
        if self.handle:
            lib().im_cuda_device_free(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Buffer:
    """MetalBuffer counterpart (crates/ironmill-metal-sys/src/buffer.rs:42-158)."""

    def __init__(self, dev: Device, nbytes: int, data: bytes | None = None):
        self.handle = C.c_void_p()
        if data is None:
            check(lib().im_cuda_buffer_alloc(dev.handle, C.c_size_t(nbytes), C.byref(self.handle)))
        else:
            check(lib().im_cuda_buffer_alloc_with_data(dev.handle, data, C.c_size_t(len(data)), C.byref(self.handle)))

    def __len__(self):
        return int(lib().im_cuda_buffer_length(self.handle))

    @property
    def ptr(self) -> int:
        return int(lib().im_cuda_buffer_ptr(self.handle) or 0)

    def write_bytes(self, data: bytes, offset: int = 0) -> None:
        check(lib().im_cuda_buffer_upload(self.handle, C.c_size_t(offset), data, C.c_size_t(len(data))))

    def read_bytes(self, nbytes: int, offset: int = 0) -> bytes:
        out = C.create_string_buffer(nbytes)
        check(lib().im_cuda_buffer_download(self.handle, C.c_size_t(offset), out, C.c_size_t(nbytes)))
        return out.raw

    def free(self):
        if self.handle:
            lib().im_cuda_buffer_free(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def quantize_affine(w: torch.Tensor, group_size: int, bit_width: int, awq: torch.Tensor | None = None):
    """GPU quantize + pack.  w fp16 [rows, K] -> (packed u8, scales f32 [rows,G], zps f32 [rows,G])."""
    assert w.is_cuda and w.dtype == torch.float16 and w.is_contiguous()
    rows = int(np.prod(w.shape[:-1])) if w.dim() > 1 else 1
    K = w.shape[-1] if w.dim() else 0
    G = -(-K // group_size) if K else 0
    total = rows * K
    nbytes = (total + 1) // 2 if bit_width == 4 else total
    packed = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
    scales = torch.empty((rows, G), dtype=torch.float32, device=w.device)
    zps = torch.empty((rows, G), dtype=torch.float32, device=w.device)
    check(lib().im_cuda_quantize_affine(vp(w), vp(awq), C.c_size_t(rows), C.c_size_t(K), C.c_int(group_size),
                                        C.c_int(bit_width), vp(packed), vp(scales), vp(zps), _stream()))
    return packed, scales, zps


class AffineWeight:
    """GPU-resident affine-quantized weight (AffineQuantizedWeight,
    crates/ironmill-inference/src/metal/weights.rs:129-147)."""

    def __init__(self, dev: Device, qdata, scales, zeros, N: int, K: int, group_size: int, bit_width: int, awq=None):
        self.dev = dev
        self.N, self.K, self.group_size, self.bit_width = N, K, group_size, bit_width
        self.handle = C.c_void_p()
        if isinstance(qdata, torch.Tensor):
            assert qdata.is_cuda and scales.is_cuda and zeros.is_cuda
            pd = IM_DTYPE_F32 if scales.dtype == torch.float32 else IM_DTYPE_F16
            assert scales.dtype == zeros.dtype and scales.is_contiguous() and zeros.is_contiguous()
            check(lib().im_cuda_affine_weight_create_dev(dev.handle, vp(qdata), vp(scales), vp(zeros), C.c_int(pd),
                                                         vp(awq), C.c_int(N), C.c_int(K), C.c_int(group_size),
                                                         C.c_int(bit_width), _stream(), C.byref(self.handle)))
            torch.cuda.current_stream().synchronize()
        else:
            qdata = np.ascontiguousarray(qdata)
            scales = np.ascontiguousarray(scales)
            zeros = np.ascontiguousarray(zeros)
            assert scales.dtype == zeros.dtype and scales.dtype in (np.float32, np.float16)
            pd = IM_DTYPE_F32 if scales.dtype == np.float32 else IM_DTYPE_F16
            if awq is not None:
                awq = np.ascontiguousarray(awq)
                assert awq.dtype == np.float16
            check(lib().im_cuda_affine_weight_create(dev.handle, vp(qdata), vp(scales), vp(zeros), C.c_int(pd), vp(awq),
                                                     C.c_int(N), C.c_int(K), C.c_int(group_size), C.c_int(bit_width),
                                                     C.byref(self.handle)))

    def nbytes(self) -> int:
        return int(lib().im_cuda_affine_weight_bytes(self.handle))

    def dequant(self) -> torch.Tensor:
        out = torch.empty((self.N, self.K), dtype=torch.float16, device=f"cuda:{self.dev.ordinal}")
        check(lib().im_cuda_affine_weight_dequant(self.handle, vp(out), _stream()))
        return out

    def free(self):
        if self.handle:
            lib().im_cuda_affine_weight_free(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _rows(x: torch.Tensor, K: int) -> int:
    assert x.is_cuda and x.dtype == torch.float16 and x.is_contiguous()
    assert x.shape[-1] == K, (x.shape, K)
    return x.numel() // K


def matvec_affine(w: AffineWeight, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    B = _rows(x, w.K)
    y = out if out is not None else torch.empty((B, w.N), dtype=torch.float16, device=x.device)
    check(lib().im_cuda_matvec_affine(w.handle, vp(x), vp(y), C.c_int(B), _stream()))
    return y


def silu_mul(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """silu_gate (crates/ironmill-inference/src/metal/shaders/activation/activation.metal): f16(SiLU(gate) * up), f32 inside."""
    assert gate.is_cuda and gate.dtype == torch.float16 and gate.is_contiguous() and up.shape == gate.shape and up.is_contiguous()
    y = out if out is not None else torch.empty_like(gate)
    check(lib().im_cuda_silu_mul(vp(gate), vp(up), vp(y), C.c_size_t(gate.numel()), _stream()))
    return y


def matmul_affine(w: AffineWeight, x: torch.Tensor, out: torch.Tensor | None = None, scratch: torch.Tensor | None = None) -> torch.Tensor:
    """Dense INT4 g128 GEMM on the tcgen05 tensor cores: y[M, N] = f16(x / awq) @ dequant(w)^T.  scratch: M * K halves."""
    M = _rows(x, w.K)
    y = out if out is not None else torch.empty((M, w.N), dtype=torch.float16, device=x.device)
    if scratch is None:
        scratch = torch.empty((M, w.K), dtype=torch.float16, device=x.device)
    check(lib().im_cuda_matmul_affine(w.handle, vp(x), vp(y), C.c_int(M), vp(scratch), _stream()))
    return y


def matvec_affine_host(w: AffineWeight, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x)
    assert x.dtype == np.float16
    B = x.size // w.K
    y = np.empty((B, w.N), dtype=np.float16)
    check(lib().im_cuda_matvec_affine_host(w.handle, vp(x), vp(y), C.c_int(B)))
    return y


def ffn_gate_up_act(gate: AffineWeight, up: AffineWeight, x: torch.Tensor, out: torch.Tensor | None = None):
    B = _rows(x, gate.K)
    y = out if out is not None else torch.empty((B, gate.N), dtype=torch.float16, device=x.device)
    check(lib().im_cuda_ffn_gate_up_act(gate.handle, up.handle, vp(x), vp(y), C.c_int(B), _stream()))
    return y


def fused_residual_norm_matvec(w: AffineWeight, a: torch.Tensor, b: torch.Tensor, gamma: torch.Tensor, eps: float,
                               want_residual: bool = True, want_normed: bool = True):
    B = _rows(a, w.K)
    assert b.shape == a.shape and b.dtype == torch.float16 and gamma.dtype == torch.float16
    y = torch.empty((B, w.N), dtype=torch.float16, device=a.device)
    res = torch.empty_like(a) if want_residual else None
    nrm = torch.empty_like(a) if want_normed else None
    check(lib().im_cuda_fused_residual_norm_matvec(w.handle, vp(a), vp(b), vp(gamma), C.c_float(eps), vp(y), vp(res),
                                                   vp(nrm), C.c_int(B), _stream()))
    return y, res, nrm


def matvec_f16(w: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    assert w.is_cuda and w.dtype == torch.float16 and w.is_contiguous() and w.dim() == 2
    N, K = w.shape
    B = _rows(x, K)
    y = torch.empty((B, N), dtype=torch.float16, device=x.device)
    check(lib().im_cuda_matvec_f16(vp(w), vp(x), vp(y), C.c_int(N), C.c_int(K), C.c_int(B), _stream()))
    return y


# ---------------------------------------------------------------- norms / embedding / RoPE
def _h16(x):
    assert x.is_cuda and x.dtype == torch.float16 and x.is_contiguous()
    return x


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    H = x.shape[-1]
    out = torch.empty_like(_h16(x))
    check(lib().im_cuda_rms_norm(vp(x), vp(_h16(gamma)), vp(out), C.c_int(H), C.c_int(x.numel() // H), C.c_float(eps), _stream()))
    return out


def fused_residual_rms_norm(a, b, gamma, eps):
    H = a.shape[-1]
    normed, residual = torch.empty_like(_h16(a)), torch.empty_like(a)
    check(lib().im_cuda_fused_residual_rms_norm(vp(a), vp(_h16(b)), vp(_h16(gamma)), vp(normed), vp(residual), C.c_int(H),
                                                C.c_int(a.numel() // H), C.c_float(eps), _stream()))
    return normed, residual


def residual_add(a, b):
    out = torch.empty_like(_h16(a))
    check(lib().im_cuda_residual_add(vp(a), vp(_h16(b)), vp(out), C.c_size_t(a.numel()), _stream()))
    return out


def embedding_norm(tokens: torch.Tensor, table: torch.Tensor, gamma: torch.Tensor, eps: float, embed_scale: float = 1.0):
    assert tokens.is_cuda and tokens.dtype in (torch.int32, torch.uint32) and tokens.is_contiguous()
    vocab, H = _h16(table).shape
    T = tokens.numel()
    normed = torch.empty((T, H), dtype=torch.float16, device=table.device)
    raw = torch.empty_like(normed)
    check(lib().im_cuda_embedding_norm(vp(tokens), vp(table), vp(_h16(gamma)), vp(normed), vp(raw), C.c_int(H), C.c_int(T),
                                       C.c_uint32(vocab), C.c_float(eps), C.c_float(embed_scale), _stream()))
    return normed, raw


def rope_table(head_dim: int, max_pos: int, theta: float, rotary_dim: int | None = None, device="cuda"):
    cos = torch.empty((max_pos, head_dim // 2), dtype=torch.float16, device=device)
    sin = torch.empty_like(cos)
    check(lib().im_cuda_rope_table(C.c_int(head_dim), C.c_int(max_pos), C.c_double(theta), C.c_int(rotary_dim or 0), vp(cos), vp(sin)))
    return cos, sin


def qk_norm_rope_(q, k, qw, kw, cos, sin, nh, nkv, hd, seq_offset, eps, rotary_dim=None):
    """In place on q [T,nh,hd] and k [T,nkv,hd]."""
    T = _h16(q).numel() // (nh * hd)
    check(lib().im_cuda_qk_norm_rope(vp(q), vp(_h16(k)), vp(_h16(qw)), vp(_h16(kw)), vp(cos), vp(sin), C.c_int(nh), C.c_int(nkv),
                                     C.c_int(hd), C.c_int(rotary_dim or hd), C.c_int(seq_offset), C.c_int(T), C.c_float(eps), _stream()))


def rope_(qk, cos, sin, heads, hd, seq_offset):
    T = _h16(qk).numel() // (heads * hd)
    check(lib().im_cuda_rope(vp(qk), vp(cos), vp(sin), C.c_int(heads), C.c_int(hd), C.c_int(seq_offset), C.c_int(T), _stream()))


# ---------------------------------------------------------------- TurboQuant
def tq_lloyd_max(dim: int, n_bits: int):
    levels = np.zeros(1 << n_bits, dtype=np.float32)
    bounds = np.zeros((1 << n_bits) - 1, dtype=np.float32)
    check(lib().im_cuda_tq_lloyd_max(C.c_int(dim), C.c_int(n_bits), vp(levels), vp(bounds)))
    return levels, bounds


def tq_generate(head_dim: int, seed: int):
    signs = np.zeros(head_dim, dtype=np.float32)
    qjl = np.zeros((head_dim, head_dim), dtype=np.float32)
    check(lib().im_cuda_tq_generate(C.c_int(head_dim), C.c_uint64(seed), vp(signs), vp(qjl)))
    return signs, qjl


class TurboQuant:
    """MetalTurboQuantModel counterpart (crates/ironmill-inference/src/metal/turboquant/mod.rs:221-287)."""

    def __init__(self, dev: Device, head_dim: int, n_bits: int, signs: np.ndarray, qjl: np.ndarray,
                 k_levels=None, k_bounds=None, v_levels=None, v_bounds=None):
        self.dev, self.head_dim, self.n_bits = dev, head_dim, n_bits
        self.handle = C.c_void_p()
        f = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)  # noqa: E731
        self._keep = [f(signs), f(qjl), f(k_levels), f(k_bounds), f(v_levels), f(v_bounds)]
        check(lib().im_cuda_tq_create(dev.handle, C.c_int(head_dim), C.c_int(n_bits), *[vp(a) for a in self._keep],
                                      C.byref(self.handle)))

    def encode(self, kv, is_k, cache, scale, r_norms, nkv, max_seq, base_pos, nseq=1, pos_dev=None):
        T = _h16(kv).numel() // (nseq * nkv * self.head_dim)
        check(lib().im_cuda_tq_encode(self.handle, vp(kv), C.c_int(int(is_k)), vp(cache), vp(scale), vp(r_norms), C.c_int(nseq),
                                      C.c_int(nkv), C.c_int(max_seq), C.c_int(base_pos), vp(pos_dev), C.c_int(T), _stream()))

    def attention(self, q, k_cache, v_cache, k_scale, v_scale, k_rnorm, attn_scale, nh, nkv, max_seq, base_pos, nseq=1,
                  pos_dev=None, num_splits=0):
        T = _h16(q).numel() // (nseq * nh * self.head_dim)
        out = torch.empty_like(q)
        check(lib().im_cuda_tq_attention(self.handle, vp(q), vp(k_cache), vp(v_cache), vp(k_scale), vp(v_scale), vp(k_rnorm),
                                         C.c_float(attn_scale), vp(out), C.c_int(nseq), C.c_int(nh), C.c_int(nkv), C.c_int(max_seq),
                                         C.c_int(base_pos), vp(pos_dev), C.c_int(T), C.c_int(num_splits), _stream()))
        return out

    def prefill_attention(self, q, k_cache, v_cache, k_scale, v_scale, k_rnorm, attn_scale, nh, nkv, max_seq, base_pos):
        """T tokens of one sequence at positions base_pos .. (rows already cached): dequantise once + causal tensor-core pass."""
        T = _h16(q).numel() // (nh * self.head_dim)
        out = torch.empty_like(q)
        dq = torch.empty(int(lib().im_cuda_tq_prefill_scratch_bytes(C.c_int(nkv), C.c_int(max_seq))), dtype=torch.uint8, device=q.device)
        check(lib().im_cuda_tq_prefill_attention(self.handle, vp(q), vp(k_cache), vp(v_cache), vp(k_scale), vp(v_scale), vp(k_rnorm),
                                                 C.c_float(attn_scale), vp(out), C.c_int(nh), C.c_int(nkv), C.c_int(max_seq), C.c_int(base_pos),
                                                 C.c_int(T), vp(dq), _stream()))
        return out

    def free(self):
        if self.handle:
            lib().im_cuda_tq_free(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def fused_residual_norm_ffn(gate: AffineWeight, up: AffineWeight, a, b, gamma, eps: float):
    """residual + RMSNorm + gate/up + SiLU in one launch -> (out [B, I], residual, normed)."""
    B = _rows(a, gate.K)
    out = torch.empty((B, gate.N), dtype=torch.float16, device=a.device)
    res, nrm = torch.empty_like(a), torch.empty_like(a)
    check(lib().im_cuda_fused_residual_norm_ffn(gate.handle, up.handle, vp(a), vp(_h16(b)), vp(_h16(gamma)), C.c_float(eps), vp(out),
                                                vp(res), vp(nrm), C.c_int(B), _stream()))
    return out, res, nrm


def tq_fused_attention(tq: "TurboQuant", qkv, nh, nkv, cos, sin, k_cache, v_cache, k_scale, v_scale, k_rnorm, attn_scale, max_seq,
                       base_pos, eps=1e-6, qw=None, kw=None, nseq=1, pos_dev=None, num_splits=0, rotary_dim=0):
    """(QK-norm +) RoPE + K/V cache write + attention from a fused QKV row [nseq*T, (nh + 2 nkv) * hd]."""
    hd = tq.head_dim
    stride = (nh + 2 * nkv) * hd
    MT = _h16(qkv).numel() // stride
    T = MT // nseq
    out = torch.empty((MT, nh * hd), dtype=torch.float16, device=qkv.device)
    qrot = torch.empty((MT, nh, 2, hd), dtype=torch.float32, device=qkv.device)
    check(lib().im_cuda_tq_fused_attention(tq.handle, vp(qkv), C.c_int(stride), C.c_int(nh * hd), C.c_int((nh + nkv) * hd), vp(qw), vp(kw),
                                           vp(cos), vp(sin), C.c_int(rotary_dim), C.c_float(eps), vp(k_cache), vp(v_cache), vp(k_scale),
                                           vp(v_scale), vp(k_rnorm), C.c_float(attn_scale), vp(qrot), vp(out), C.c_int(nseq), C.c_int(nh),
                                           C.c_int(nkv), C.c_int(max_seq), C.c_int(base_pos), vp(pos_dev), C.c_int(T), C.c_int(num_splits),
                                           _stream()))
    return out


def tq_attention_static(tq: "TurboQuant", q, k_cache, v_cache, k_scale, v_scale, k_rnorm, attn_scale, nh, nkv, max_seq, base_pos,
                        nseq=1, pos_dev=None, num_splits=0):
    """Attention through the entry point that allocates nothing (split partials in the library's built-in array)."""
    T = _h16(q).numel() // (nseq * nh * tq.head_dim)
    out = torch.empty_like(q)
    check(lib().im_cuda_tq_attention_static(tq.handle, vp(q), vp(k_cache), vp(v_cache), vp(k_scale), vp(v_scale), vp(k_rnorm),
                                            C.c_float(attn_scale), vp(out), C.c_int(nseq), C.c_int(nh), C.c_int(nkv), C.c_int(max_seq),
                                            C.c_int(base_pos), vp(pos_dev), C.c_int(T), C.c_int(num_splits), _stream()))
    return out


def kv_scatter_f16(proj, cache, nseq, T, nkv, max_seq, base_pos, pos_dev=None):
    """kv_scatter (shaders/kv/kv_scatter.metal:20-42): proj fp16 [nseq*T, nkv, 128] -> cache fp16 [nseq, nkv, max_seq, 128]."""
    check(lib().im_cuda_kv_scatter_f16(vp(proj), vp(cache), C.c_int(nseq), C.c_int(T), C.c_int(nkv), C.c_int(128), C.c_int(max_seq),
                                       C.c_int(base_pos), vp(pos_dev), None, _stream()))


def sdpa_f16(dev: "Device", q, k_cache, v_cache, scale, nh, nkv, max_seq, base_pos, nseq=1, pos_dev=None, num_splits=0):
    """fp16-KV attention (fused_sdpa / prefill_attention_v2 / fused_sdpa_split + reduce): q fp16 [nseq*T, nh, 128]."""
    T = _h16(q).numel() // (nseq * nh * 128)
    out = torch.empty_like(q)
    splits = num_splits if num_splits > 0 else 64
    nbytes = int(lib().im_cuda_sdpa_f16_scratch_bytes(C.c_int(nseq), C.c_int(T), C.c_int(nh), C.c_int(splits)))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    check(lib().im_cuda_sdpa_f16(dev.handle, vp(q), vp(k_cache), vp(v_cache), vp(out), C.c_int(nseq), C.c_int(nh), C.c_int(nkv), C.c_int(128),
                                 C.c_int(max_seq), C.c_int(base_pos), vp(pos_dev), C.c_int(T), C.c_float(scale), C.c_int(num_splits),
                                 vp(scratch), C.c_size_t(nbytes), _stream()))
    return out

