// Per-group affine quantization + INT4 packing on the GPU, bit-exact with the reference's
// CPU quantizer: quantize_affine / emit_per_group
// (crates/mil-rs/src/ir/passes/affine_quantize.rs:256-298,420-453), pack_int4
// (crates/mil-rs/src/ir/passes/int4_pack.rs:20-34) and the AWQ column pre-scale
// (crates/ironmill-compile/src/weights/quantized.rs:925-940).
//
// Every float operation is an explicit round-to-nearest intrinsic so that no multiply-add is
// contracted; roundf() is round-half-away-from-zero like Rust's f32::round.
#include <float.h>

#include "common.cuh"

namespace im {

__device__ __forceinline__ float load_weight(const __half *w, const __half *awq, size_t idx, size_t col) {
    float x = __half2float(w[idx]);
    if (awq) x = __fmul_rn(x, __half2float(awq[col]));
    return x;
}

// One warp per (row, group): min/max over the finite values, then scale and zero point.
// The CPU loop keeps the first of equal extrema (strict compares); that only matters for
// the sign of a zero, and is reproduced by carrying the element index through the reduction.
__global__ void quantize_params_kernel(const __half *__restrict__ w, const __half *__restrict__ awq,
                                       size_t rows, size_t K, int gs, int G, float qmax,
                                       float *__restrict__ scales, float *__restrict__ zps) {
    size_t gid = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    int lane = threadIdx.x & 31;
    if (gid >= rows * (size_t)G) return;
    size_t r = gid / G;
    int g = (int)(gid % G);
    size_t c0 = (size_t)g * gs, c1 = c0 + gs < K ? c0 + gs : K;

    float mn = INFINITY, mx = -INFINITY;
    unsigned imn = 0xffffffffu, imx = 0xffffffffu;
    for (size_t c = c0 + lane; c < c1; c += 32) {
        float x = load_weight(w, awq, r * K + c, c);
        if (isfinite(x)) {
            if (x < mn) { mn = x; imn = (unsigned)(c - c0); }
            if (x > mx) { mx = x; imx = (unsigned)(c - c0); }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float omn = __shfl_xor_sync(0xffffffffu, mn, o);
        unsigned oimn = __shfl_xor_sync(0xffffffffu, imn, o);
        float omx = __shfl_xor_sync(0xffffffffu, mx, o);
        unsigned oimx = __shfl_xor_sync(0xffffffffu, imx, o);
        if (omn < mn || (omn == mn && oimn < imn)) { mn = omn; imn = oimn; }
        if (omx > mx || (omx == mx && oimx < imx)) { mx = omx; imx = oimx; }
    }
    if (lane == 0) {
        float scale, zp;
        if (!isfinite(mn) || !isfinite(mx)) {
            scale = 1.0f;
            zp = 0.0f;
        } else if (fabsf(__fsub_rn(mx, mn)) < FLT_EPSILON) {
            scale = 1.0f;
            zp = roundf(-mn);
        } else {
            scale = __fdiv_rn(__fsub_rn(mx, mn), qmax);
            zp = roundf(__fdiv_rn(-mn, scale));
        }
        scales[gid] = scale;
        zps[gid] = zp;
    }
}

// A group without any finite value quantizes to all zeros (the CPU routine returns early with
// a zero vector); a non-finite element of any other group saturates through the clamp.  Only
// non-finite elements take the rescan, so the common path stays one pass.
__device__ __noinline__ bool group_has_finite(const __half *w, const __half *awq, size_t row_base, size_t c0, size_t c1) {
    for (size_t c = c0; c < c1; c++)
        if (isfinite(load_weight(w, awq, row_base + c, c))) return true;
    return false;
}

__device__ __forceinline__ unsigned quantize_elem(const __half *w, const __half *awq, size_t i, size_t K, int gs, int G,
                                                  const float *scales, const float *zps, float qmax);

__device__ __forceinline__ unsigned quantize_one(float x, float scale, float zp, float qmax) {
    float t = roundf(__fadd_rn(__fdiv_rn(x, scale), zp));
    if (t != t) return 0u;  // NaN saturates to 0 like Rust's `as u8`
    t = fminf(fmaxf(t, 0.0f), qmax);
    return (unsigned)t;
}

__device__ __forceinline__ unsigned quantize_elem(const __half *w, const __half *awq, size_t i, size_t K, int gs, int G,
                                                  const float *scales, const float *zps, float qmax) {
    const size_t r = i / K, c = i % K;
    const size_t g = c / gs, pi = r * G + g;
    const float x = load_weight(w, awq, i, c);
    if (!isfinite(x)) {
        const size_t c0 = g * gs, c1 = c0 + gs < K ? c0 + gs : K;
        if (!group_has_finite(w, awq, r * K, c0, c1)) return 0u;
    }
    return quantize_one(x, scales[pi], zps[pi], qmax);
}

// 4-bit: one thread per output byte = flat element pair (2p, 2p+1); the pair may straddle
// groups or rows when K is odd, so each element looks up its own group.
__global__ void quantize_codes_int4_kernel(const __half *__restrict__ w, const __half *__restrict__ awq,
                                           size_t total, size_t K, int gs, int G,
                                           const float *__restrict__ scales, const float *__restrict__ zps,
                                           uint8_t *__restrict__ packed) {
    size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t nbytes = (total + 1) / 2;
    if (p >= nbytes) return;
    unsigned byte = 0;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        size_t i = 2 * p + h;
        if (i < total) {
            unsigned q = quantize_elem(w, awq, i, K, gs, G, scales, zps, 15.0f);
            byte |= (q & 0xFu) << (4 * h);
        }
    }
    packed[p] = (uint8_t)byte;
}

__global__ void quantize_codes_int8_kernel(const __half *__restrict__ w, const __half *__restrict__ awq,
                                           size_t total, size_t K, int gs, int G,
                                           const float *__restrict__ scales, const float *__restrict__ zps,
                                           uint8_t *__restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    out[i] = (uint8_t)quantize_elem(w, awq, i, K, gs, G, scales, zps, 255.0f);
}

}  // namespace im

IM_EXPORT int im_cuda_quantize_affine(const void *w_dev, const void *awq_dev, size_t rows, size_t K,
                                      int group_size, int bit_width, void *packed_dev, float *scales_dev,
                                      float *zps_dev, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(bit_width == 4 || bit_width == 8, "bit_width must be 4 or 8, got %d", bit_width);
    IM_REQUIRE(group_size > 0, "group_size must be positive");
    size_t total = rows * K;
    if (total == 0) return IM_OK;  // empty input: nothing to write
    IM_REQUIRE(w_dev && packed_dev && scales_dev && zps_dev, "NULL device pointer");
    size_t G = (K + group_size - 1) / group_size;
    IM_REQUIRE(G <= 0x7fffffff && rows * G / 8 + 1 <= 0x7fffffff, "tensor too large");
    cudaStream_t st = im::as_stream(stream);
    const __half *w = static_cast<const __half *>(w_dev);
    const __half *awq = static_cast<const __half *>(awq_dev);
    size_t ngroups = rows * G;
    const int warps_per_block = 8;
    im::quantize_params_kernel<<<(unsigned)((ngroups + warps_per_block - 1) / warps_per_block), warps_per_block * 32, 0, st>>>(
        w, awq, rows, K, group_size, (int)G, bit_width == 4 ? 15.0f : 255.0f, scales_dev, zps_dev);
    if (bit_width == 4) {
        size_t nbytes = (total + 1) / 2;
        im::quantize_codes_int4_kernel<<<(unsigned)((nbytes + 255) / 256), 256, 0, st>>>(
            w, awq, total, K, group_size, (int)G, scales_dev, zps_dev, static_cast<uint8_t *>(packed_dev));
    } else {
        im::quantize_codes_int8_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            w, awq, total, K, group_size, (int)G, scales_dev, zps_dev, static_cast<uint8_t *>(packed_dev));
    }
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
    IM_GUARD_END
}
