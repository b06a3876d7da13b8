// Norm / embedding / RoPE kernels of the decode path (fp16 in and out, f32 arithmetic):
//   rms_norm                 crates/ironmill-inference/src/metal/shaders/norm/normalization.metal:19-57
//   fused_residual_rms_norm  .../shaders/norm/fused_residual_norm.metal:33-75
//   residual_add             .../shaders/elementwise/elementwise.metal:14-23
//   fused_embedding_norm     .../shaders/norm/fused_embedding_norm.metal:29-72
//   fused_qk_norm_rope       .../shaders/norm/fused_qk_norm_rope.metal:43-124
//   rope                     .../shaders/rope/rope.metal:21-60
//   RoPE table               crates/ironmill-core/src/rope.rs:22-49 (host, f64)
// One CTA per token (per head for the head-wise kernels); rows are read with 128-bit loads when
// the row length allows it.  Positions can come from a device word so that a captured CUDA
// graph replays with a moving sequence position.
#include <math.h>

#include <vector>

#include "common.cuh"

namespace im {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float *sh) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();  // sh may still be read from a previous call
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; w++) t += sh[w];
    return t;
}

// MODE 0: out = norm(x); MODE 1: r = a + b, residual = f16(r), out = norm(r) from the unrounded sum.
template <int MODE>
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const __half *__restrict__ a, const __half *__restrict__ b,
                                                                const __half *__restrict__ gamma, __half *__restrict__ normed,
                                                                __half *__restrict__ residual, int H, float eps) {
    __shared__ float sh[32];
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = __half2float(a[base + i]);
        if (MODE == 1) {
            v += __half2float(b[base + i]);
            residual[base + i] = __float2half_rn(v);
        }
        ss += v * v;
    }
    const float tot = block_sum(ss, sh);
    const float rms_inv = rsqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = __half2float(a[base + i]);
        if (MODE == 1) v += __half2float(b[base + i]);
        normed[base + i] = __float2half_rn(v * rms_inv * __half2float(gamma[i]));
    }
}

__global__ void residual_add_kernel(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(__half2float(a[i]) + __half2float(b[i]));
}

__global__ void __launch_bounds__(kNormThreads) embedding_norm_kernel(const uint32_t *__restrict__ tokens, const __half *__restrict__ table,
                                                                      const __half *__restrict__ gamma, __half *__restrict__ normed,
                                                                      __half *__restrict__ raw, int H, uint32_t vocab, float eps,
                                                                      float embed_scale) {
    __shared__ float sh[32];
    pdl_trigger();
    pdl_wait();
    const uint32_t tok = tokens[blockIdx.x];
    const bool valid = tok < vocab;
    const size_t src = (size_t)tok * H, dst = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = valid ? __half2float(table[src + i]) * embed_scale : 0.0f;
        raw[dst + i] = __float2half_rn(v);
        ss += v * v;
    }
    const float tot = block_sum(ss, sh);
    const float rms_inv = rsqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = valid ? __half2float(table[src + i]) * embed_scale : 0.0f;
        normed[dst + i] = __float2half_rn(v * rms_inv * __half2float(gamma[i]));
    }
}

// grid (nh + nkv [+ nkv], T), one CTA per head.  with_norm = 0 gives plain RoPE (Llama).
// Reads q/k (and optionally v) with a per-token stride, writes dense [T, heads, hd] outputs;
// input and output may be the same buffer.  The optional third group of CTAs copies V heads
// so that a fused QKV projection row can be split into dense Q, K and V in this one launch.
__global__ void qk_norm_rope_kernel(const QkRopeArgs a) {
    __shared__ float sh[32];
    const int slot = blockIdx.x, t = blockIdx.y;
    const int hd = a.hd;
    if (slot >= a.nh + a.nkv) {  // V copy
        const int h = slot - a.nh - a.nkv;
        const __half *src = a.v_in + (size_t)t * a.v_stride + (size_t)h * hd;
        __half *dst = a.v_out + ((size_t)t * a.nkv + h) * hd;
        for (int d = threadIdx.x; d < hd; d += blockDim.x) dst[d] = src[d];
        return;
    }
    const bool is_q = slot < a.nh;
    const int h = is_q ? slot : slot - a.nh, heads = is_q ? a.nh : a.nkv;
    const __half *src = (is_q ? a.q_in + (size_t)t * a.q_stride : a.k_in + (size_t)t * a.k_stride) + (size_t)h * hd;
    __half *dst = (is_q ? a.q_out : a.k_out) + ((size_t)t * heads + h) * hd;
    const __half *w = is_q ? a.qw : a.kw;
    float rms_inv = 1.0f;
    if (a.with_norm) {
        float ss = 0.0f;
        for (int d = threadIdx.x; d < hd; d += blockDim.x) {
            const float v = __half2float(src[d]);
            ss += v * v;
        }
        const float tot = block_sum(ss, sh);
        rms_inv = rsqrtf(tot / (float)hd + a.eps);
    }
    const int half_rot = a.rotary_dim / 2, half_dim = hd / 2;
    const int seq = t / a.tokens_per_seq, tt = t % a.tokens_per_seq;
    const int pos = a.seq_offset + (a.pos_dev ? a.pos_dev[seq] : 0) + tt;
    for (int d = threadIdx.x; d < half_rot; d += blockDim.x) {
        float lo = __half2float(src[d]), hi = __half2float(src[d + half_rot]);
        if (a.with_norm) {
            lo = lo * rms_inv * __half2float(w[d]);
            hi = hi * rms_inv * __half2float(w[d + half_rot]);
        }
        const float c = __half2float(a.cosc[(size_t)pos * half_dim + d]), s = __half2float(a.sinc[(size_t)pos * half_dim + d]);
        dst[d] = __float2half_rn(lo * c - hi * s);
        dst[d + half_rot] = __float2half_rn(lo * s + hi * c);
    }
    for (int d = threadIdx.x + a.rotary_dim; d < hd; d += blockDim.x) {
        float v = __half2float(src[d]);
        if (a.with_norm) v = v * rms_inv * __half2float(w[d]);
        dst[d] = __float2half_rn(v);
    }
}

int launch_qk_rope(const QkRopeArgs &a, int T, cudaStream_t st) {
    const int slots = a.nh + a.nkv + (a.v_in ? a.nkv : 0);
    if (T == 0 || slots == 0) return IM_OK;
    const int threads = a.hd >= 256 ? 128 : (a.hd / 2 >= 32 ? (a.hd / 2 + 31) / 32 * 32 : 32);
    dim3 grid(slots, T);
    qk_norm_rope_kernel<<<grid, threads, 0, st>>>(a);
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
}

}  // namespace im

using namespace im;

IM_EXPORT int im_cuda_rms_norm(const void *x_dev, const void *gamma_dev, void *out_dev, int H, int T, float eps, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(x_dev && gamma_dev && out_dev, "bad argument");
    IM_REQUIRE(H > 0 && T >= 0, "bad shape");
    if (T == 0) return IM_OK;
    IM_CUDA_CHECK(launch_k(rms_norm_kernel<0>, dim3(T), dim3(kNormThreads), 0, as_stream(stream), static_cast<const __half *>(x_dev),
                           (const __half *)nullptr, static_cast<const __half *>(gamma_dev), static_cast<__half *>(out_dev),
                           (__half *)nullptr, H, eps));
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_fused_residual_rms_norm(const void *a_dev, const void *b_dev, const void *gamma_dev, void *normed_dev,
                                              void *residual_dev, int H, int T, float eps, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(a_dev && b_dev && gamma_dev && normed_dev && residual_dev, "bad argument");
    IM_REQUIRE(H > 0 && T >= 0, "bad shape");
    if (T == 0) return IM_OK;
    IM_CUDA_CHECK(launch_k(rms_norm_kernel<1>, dim3(T), dim3(kNormThreads), 0, as_stream(stream), static_cast<const __half *>(a_dev),
                           static_cast<const __half *>(b_dev), static_cast<const __half *>(gamma_dev), static_cast<__half *>(normed_dev),
                           static_cast<__half *>(residual_dev), H, eps));
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_residual_add(const void *a_dev, const void *b_dev, void *out_dev, size_t n, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(a_dev && b_dev && out_dev, "bad argument");
    if (n == 0) return IM_OK;
    IM_CUDA_CHECK(launch_k(residual_add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, as_stream(stream),
                           static_cast<const __half *>(a_dev), static_cast<const __half *>(b_dev), static_cast<__half *>(out_dev), n));
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_embedding_norm(const uint32_t *tokens_dev, const void *table_dev, const void *gamma_dev, void *normed_dev,
                                     void *raw_dev, int H, int T, uint32_t vocab, float eps, float embed_scale, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(tokens_dev && table_dev && gamma_dev && normed_dev && raw_dev, "bad argument");
    IM_REQUIRE(H > 0 && T >= 0, "bad shape");
    if (T == 0) return IM_OK;
    IM_CUDA_CHECK(launch_k(embedding_norm_kernel, dim3(T), dim3(kNormThreads), 0, as_stream(stream), tokens_dev,
                           static_cast<const __half *>(table_dev), static_cast<const __half *>(gamma_dev),
                           static_cast<__half *>(normed_dev), static_cast<__half *>(raw_dev), H, vocab, eps, embed_scale));
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_qk_norm_rope(void *q_dev, void *k_dev, const void *q_norm_w_dev, const void *k_norm_w_dev, const void *cos_dev,
                                   const void *sin_dev, int nh, int nkv, int head_dim, int rotary_dim, int seq_offset, int T, float eps,
                                   void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(q_dev && k_dev && q_norm_w_dev && k_norm_w_dev && cos_dev && sin_dev, "bad argument");
    IM_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim, "bad head_dim / rotary_dim");
    QkRopeArgs a{};
    a.q_in = a.q_out = static_cast<__half *>(q_dev);
    a.k_in = a.k_out = static_cast<__half *>(k_dev);
    a.q_stride = nh * head_dim;
    a.k_stride = nkv * head_dim;
    a.qw = static_cast<const __half *>(q_norm_w_dev);
    a.kw = static_cast<const __half *>(k_norm_w_dev);
    a.cosc = static_cast<const __half *>(cos_dev);
    a.sinc = static_cast<const __half *>(sin_dev);
    a.nh = nh; a.nkv = nkv; a.hd = head_dim; a.rotary_dim = rotary_dim ? rotary_dim : head_dim;
    a.seq_offset = seq_offset; a.tokens_per_seq = T > 0 ? T : 1; a.eps = eps; a.with_norm = 1;
    return launch_qk_rope(a, T, as_stream(stream));
    IM_GUARD_END
}

IM_EXPORT int im_cuda_rope(void *qk_dev, const void *cos_dev, const void *sin_dev, int heads, int head_dim, int seq_offset, int T,
                           void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(qk_dev && cos_dev && sin_dev, "bad argument");
    IM_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "bad head_dim");
    QkRopeArgs a{};
    a.q_in = a.q_out = static_cast<__half *>(qk_dev);
    a.q_stride = heads * head_dim;
    a.cosc = static_cast<const __half *>(cos_dev);
    a.sinc = static_cast<const __half *>(sin_dev);
    a.nh = heads; a.nkv = 0; a.hd = head_dim; a.rotary_dim = head_dim;
    a.seq_offset = seq_offset; a.tokens_per_seq = T > 0 ? T : 1; a.with_norm = 0;
    return launch_qk_rope(a, T, as_stream(stream));
    IM_GUARD_END
}

IM_EXPORT int im_cuda_rope_table(int head_dim, int max_pos, double theta, int rotary_dim, void *cos_dev, void *sin_dev) {
    IM_GUARD_BEGIN
    IM_REQUIRE(cos_dev && sin_dev, "bad argument");
    IM_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && max_pos > 0, "bad shape");
    const int half = head_dim / 2, rd = rotary_dim ? rotary_dim : head_dim, rh = rd / 2;
    std::vector<__half> c((size_t)max_pos * half), s((size_t)max_pos * half);
    std::vector<double> freq(half);
    for (int i = 0; i < rh && i < half; i++) freq[i] = 1.0 / pow(theta, 2.0 * (double)i / (double)rd);
    for (int p = 0; p < max_pos; p++)
        for (int i = 0; i < half; i++) {
            if (i < rh) {
                const double ang = (double)p * freq[i];
                c[(size_t)p * half + i] = __double2half(cos(ang));
                s[(size_t)p * half + i] = __double2half(sin(ang));
            } else {
                c[(size_t)p * half + i] = __double2half(1.0);
                s[(size_t)p * half + i] = __double2half(0.0);
            }
        }
    IM_CUDA_CHECK(cudaMemcpy(cos_dev, c.data(), c.size() * sizeof(__half), cudaMemcpyHostToDevice));
    IM_CUDA_CHECK(cudaMemcpy(sin_dev, s.data(), s.size() * sizeof(__half), cudaMemcpyHostToDevice));
    return IM_OK;
    IM_GUARD_END
}
