// HBM-streaming affine-quantized matvec family for decode (batch < 16):
//   plain projection            superblock_matvec_int4 / _int8
//       (crates/ironmill-inference/src/metal/shaders/quantized/affine_matvec.metal:16-111,123-189)
//   fused gate+up+SiLU          superblock_fused_ffn_gate_up_act_int4
//       (.../shaders/quantized/affine_fused.metal:9-108, affine_batched.metal:5-91)
//   fused residual+RMSNorm+matvec  superblock_fused_residual_norm_affine_matvec_int4
//       (.../shaders/norm/superblock_fused_norm.metal:21-124)
// all with the (q - z) * s dequant of crates/ironmill-core/src/dequant.rs:129-139.
//
// Design (B200): the weights are read exactly once with 128-bit streaming loads, one warp
// per group of rows, lanes side by side along K (512 contiguous bytes per warp load).  B200
// delivers ~23 weight bytes per SM clock, i.e. ~46 nibbles, so the inner loop may spend
// about one integer instruction per nibble.  The activation vector is therefore
// block-quantised once per CTA to 16-bit integers with one scale per 128-element group
// (error 2^-16 of the group maximum, far below the fp16 resolution of x itself), split into
// a signed high byte and an unsigned low byte, and staged in shared memory in the lane order
// of the weight loads.  Eight nibbles then cost 3 unpack operations and 4 dp4a, with exact
// integer accumulation inside a group, and one float fix-up per 32 nibbles:
//   sum_k x_k (q_k - z) s  =  s * sx * ( sum_k xi_k q_k  -  z * sum_k xi_k ).
// Warp shuffles reduce the lanes; shared memory reduces warps that split K.
#include <new>

#include "common.cuh"

namespace im {

constexpr int kGroup = 128;     // fast-path group size
constexpr int kWarps = 8;       // warps per CTA
constexpr int kThreads = kWarps * 32;

enum MatvecMode { kPlain = 0, kGateUpAct = 1, kResidualNorm = 2, kResNormGateUp = 3 };

struct MatvecParams {
    const uint8_t *codes0;  // plain / gate rows
    const __half2 *sz0;
    const uint8_t *codes1;  // up rows (kGateUpAct)
    const __half2 *sz1;
    const __half *awq;      // [K] or nullptr
    const __half *x;        // [B,K] (plain, gate-up) or `a` (residual-norm)
    const __half *b;        // residual-norm: second addend
    const __half *gamma;    // residual-norm: norm weight
    __half *y;              // [B,N]
    __half *residual_out;   // residual-norm side outputs (nullable)
    __half *normed_out;
    float eps;
    int N, K, G;
    int ksplit;             // warps of a CTA that share a row group along K
};

template <int BITS>
struct Lay {
    static constexpr int kElemsPerLane = BITS == 4 ? 32 : 16;   // one 16-byte load
    static constexpr int kChunk = kElemsPerLane * 32;           // elements per warp iteration
    static constexpr int kXV = BITS == 4 ? 4 : 2;               // uint4 of staged x per lane per chunk
};

__device__ __forceinline__ unsigned pack4(int a, int b, int c, int d) {
    return (unsigned)(a & 0xff) | ((unsigned)(b & 0xff) << 8) | ((unsigned)(c & 0xff) << 16) | ((unsigned)(d & 0xff) << 24);
}

// Block-quantise one batch row of activations into shared memory.
// A half-warp owns one 128-element group: 8 elements per lane.
template <int BITS, int MODE>
__device__ __forceinline__ float stage_activations(const MatvecParams &p, int b, uint4 *xq, float2 *meta) {
    const int K = p.K;
    const int lane = threadIdx.x & 31, hl = lane & 15, warp = threadIdx.x >> 5;
    float sq = 0.0f;
    // Two groups per warp pass; the trip count is uniform across the warp because the
    // half-warp shuffles below are issued with a full mask.
    for (int g0 = warp * 2; g0 < p.G; g0 += kWarps * 2) {
        const int g = g0 + (lane >> 4);
        const bool live = g < p.G;
        const int k = (live ? g : g0) * kGroup + hl * 8;
        float v[8];
        {
            uint4 raw = *reinterpret_cast<const uint4 *>(p.x + (size_t)b * K + k);
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 f = __half22float2(h[i]);
                v[2 * i] = f.x;
                v[2 * i + 1] = f.y;
            }
        }
        if (MODE == kResidualNorm) {
            uint4 rb = *reinterpret_cast<const uint4 *>(p.b + (size_t)b * K + k);
            uint4 rg = *reinterpret_cast<const uint4 *>(p.gamma + k);
            const __half2 *hb = reinterpret_cast<const __half2 *>(&rb);
            const __half2 *hg = reinterpret_cast<const __half2 *>(&rg);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 fb = __half22float2(hb[i]), fg = __half22float2(hg[i]);
                float r0 = v[2 * i] + fb.x, r1 = v[2 * i + 1] + fb.y;
                if (live) sq += r0 * r0 + r1 * r1;
                v[2 * i] = r0 * fg.x;
                v[2 * i + 1] = r1 * fg.y;
            }
        }
        if (p.awq) {
            uint4 ra = *reinterpret_cast<const uint4 *>(p.awq + k);
            const __half2 *ha = reinterpret_cast<const __half2 *>(&ra);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 fa = __half22float2(ha[i]);
                v[2 * i] = v[2 * i] / fa.x;
                v[2 * i + 1] = v[2 * i + 1] / fa.y;
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float sx = amax > 0.0f ? amax * (1.0f / 32767.0f) : 1.0f;
        const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
        int xi[8], hi[8], lo[8], lsum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            xi[i] = __float2int_rn(v[i] * inv);
            xi[i] = max(-32767, min(32767, xi[i]));
            lsum += xi[i];
            hi[i] = xi[i] >> 8;
            lo[i] = xi[i] & 0xff;
        }
        constexpr int kChunk = Lay<BITS>::kChunk, kEpl = Lay<BITS>::kElemsPerLane, kXV = Lay<BITS>::kXV;
        const int c = k / kChunk, kl = k % kChunk, ldst = kl / kEpl;
        if (BITS == 4) {
            const int j = (kl % kEpl) / 8;
            if (live) xq[(c * kXV + j) * 32 + ldst] =
                make_uint4(pack4(hi[0], hi[2], hi[4], hi[6]), pack4(hi[1], hi[3], hi[5], hi[7]),
                           pack4(lo[0], lo[2], lo[4], lo[6]), pack4(lo[1], lo[3], lo[5], lo[7]));
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
            if (live && (hl & 3) == 0) meta[c * 32 + ldst] = make_float2(sx, (float)lsum);
        } else {
            const int j = (kl % kEpl) / 8;
            if (live) xq[(c * kXV + j) * 32 + ldst] =
                make_uint4(pack4(hi[0], hi[1], hi[2], hi[3]), pack4(lo[0], lo[1], lo[2], lo[3]),
                           pack4(hi[4], hi[5], hi[6], hi[7]), pack4(lo[4], lo[5], lo[6], lo[7]));
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
            if (live && (hl & 1) == 0) meta[c * 32 + ldst] = make_float2(sx, (float)lsum);
        }
    }
    return sq;
}

template <int BITS>
__device__ __forceinline__ int dot_lane(const uint4 &w, const uint4 *xv) {
    int hi = 0, lo = 0;
    const unsigned ww[4] = {w.x, w.y, w.z, w.w};
    if (BITS == 4) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const unsigned e = ww[j] & 0x0F0F0F0Fu, o = (ww[j] >> 4) & 0x0F0F0F0Fu;
            hi = dp4a_us(e, xv[j].x, hi);
            hi = dp4a_us(o, xv[j].y, hi);
            lo = dp4a_uu(e, xv[j].z, lo);
            lo = dp4a_uu(o, xv[j].w, lo);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            hi = dp4a_us(ww[2 * j], xv[j].x, hi);
            lo = dp4a_uu(ww[2 * j], xv[j].y, lo);
            hi = dp4a_us(ww[2 * j + 1], xv[j].z, hi);
            lo = dp4a_uu(ww[2 * j + 1], xv[j].w, lo);
        }
    }
    return hi * 256 + lo;
}

// R = rows per warp (per weight matrix), NB = batch rows per launch.
template <int BITS, int MODE, int R, int NB>
__global__ void __launch_bounds__(kThreads) matvec_kernel(const MatvecParams p) {
    constexpr int kChunk = Lay<BITS>::kChunk, kEpl = Lay<BITS>::kElemsPerLane, kXV = Lay<BITS>::kXV;
    constexpr int RS = MODE == kGateUpAct ? 2 * R : R;  // row streams per warp
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = p.K, N = p.N, G = p.G;
    const int nchunks = (K + kChunk - 1) / kChunk;
    uint4 *xq = reinterpret_cast<uint4 *>(smem_raw);                               // [NB][nchunks*kXV*32]
    float2 *meta = reinterpret_cast<float2 *>(xq + (size_t)NB * nchunks * kXV * 32);  // [NB][nchunks*32]
    float *red = reinterpret_cast<float *>(meta + (size_t)NB * nchunks * 32);      // [kWarps][RS*NB] + [kWarps] + 1

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ksplit = p.ksplit;
    const int rg = warp / ksplit, kw = warp % ksplit;  // row group of the CTA, K share
    const int rgs = kWarps / ksplit;
    const size_t row_bytes = (size_t)K * BITS / 8;

    // One work item = one 16-byte weight load per row stream (plus its scale/zero pair).
    struct Item {
        uint4 wv[RS];
        __half2 szv[RS];
    };
    const int rows_per_tile = rgs * R;
    const int ntiles = (N + rows_per_tile - 1) / rows_per_tile;
    auto load_item = [&](int tile, int c, Item &it) {
        const int k0 = c * kChunk + lane * kEpl;
        if (k0 < K) {
            const int n0 = tile * rows_per_tile + rg * R;
#pragma unroll
            for (int t = 0; t < RS; t++) {
                const int n = min(n0 + (t % R), N - 1);  // clamped rows compute but never store
                const bool second = MODE == kGateUpAct && t >= R;
                it.wv[t] = ldg_stream_v4((second ? p.codes1 : p.codes0) + (size_t)n * row_bytes + (size_t)k0 * BITS / 8);
                it.szv[t] = (second ? p.sz1 : p.sz0)[(size_t)n * G + k0 / kGroup];
            }
        }
    };

    // The first weight loads are issued before the activations are staged, so that the HBM
    // pipe fills while the CTA quantises x.
    Item cur, nxt;
    int tile = blockIdx.x, c = kw;
    if (tile < ntiles && c < nchunks) load_item(tile, c, cur);

    // ---- stage activations (once per CTA) ----
    float sq_tot[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) {
        float sq = stage_activations<BITS, MODE>(p, b, xq + (size_t)b * nchunks * kXV * 32, meta + (size_t)b * nchunks * 32);
        sq_tot[b] = 0.0f;
        if (MODE == kResidualNorm) {
            sq = warp_sum(sq);
            float *rs = red + kWarps * RS * NB;
            if (lane == 0) rs[warp] = sq;
            __syncthreads();
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) t += rs[w];
            sq_tot[b] = t;
            __syncthreads();
        }
    }
    __syncthreads();

    float rms_inv[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) rms_inv[b] = MODE == kResidualNorm ? rsqrtf(sq_tot[b] / (float)K + p.eps) : 1.0f;

    // Side outputs of the fused residual+norm form, written by CTA 0 only
    // (they must not alias a or b: other CTAs are still reading those).
    if (MODE == kResidualNorm && blockIdx.x == 0) {
        for (int b = 0; b < NB; b++)
            for (int k = threadIdx.x; k < K; k += kThreads) {
                float r = __half2float(p.x[(size_t)b * K + k]) + __half2float(p.b[(size_t)b * K + k]);
                if (p.residual_out) p.residual_out[(size_t)b * K + k] = __float2half_rn(r);
                if (p.normed_out) p.normed_out[(size_t)b * K + k] = __float2half_rn(r * rms_inv[b] * __half2float(p.gamma[k]));
            }
    }

    for (; tile < ntiles; tile += gridDim.x) {
        const int n0 = tile * rows_per_tile + rg * R;
        float res[RS][NB];
#pragma unroll
        for (int t = 0; t < RS; t++)
#pragma unroll
            for (int b = 0; b < NB; b++) res[t][b] = 0.0f;

        for (c = kw; c < nchunks; c += ksplit) {
            // prefetch the next item of this warp (next chunk, or first chunk of the next tile)
            int c2 = c + ksplit, tile2 = tile;
            if (c2 >= nchunks) {
                c2 = kw;
                tile2 = tile + gridDim.x;
            }
            if (tile2 < ntiles) load_item(tile2, c2, nxt);

            const int k0 = c * kChunk + lane * kEpl;
            if (k0 < K) {
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const uint4 *xb = xq + ((size_t)b * nchunks + c) * kXV * 32 + lane;
                    uint4 xv[kXV];
#pragma unroll
                    for (int v = 0; v < kXV; v++) xv[v] = xb[v * 32];
                    const float2 m = meta[((size_t)b * nchunks + c) * 32 + lane];
#pragma unroll
                    for (int t = 0; t < RS; t++) {
                        const float f = (float)dot_lane<BITS>(cur.wv[t], xv);
                        const float2 s_z = __half22float2(cur.szv[t]);
                        res[t][b] = fmaf(s_z.x * m.x, fmaf(-s_z.y, m.y, f), res[t][b]);
                    }
                }
            }
            cur = nxt;
        }

#pragma unroll
        for (int t = 0; t < RS; t++)
#pragma unroll
            for (int b = 0; b < NB; b++) res[t][b] = warp_sum(res[t][b]);

        if (ksplit > 1) {
            __syncthreads();  // previous tile's readers are done with `red`
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < RS; t++)
#pragma unroll
                    for (int b = 0; b < NB; b++) red[(warp * RS + t) * NB + b] = res[t][b];
            }
            __syncthreads();
            if (kw == 0) {
#pragma unroll
                for (int t = 0; t < RS; t++)
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        float s = 0.0f;
                        for (int w = 0; w < ksplit; w++) s += red[((rg * ksplit + w) * RS + t) * NB + b];
                        res[t][b] = s;
                    }
            }
        }
        if (kw == 0 && lane == 0) {
#pragma unroll
            for (int t = 0; t < R; t++) {
                const int n = n0 + t;
                if (n < N) {
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        float out;
                        if (MODE == kGateUpAct) {
                            const float g = res[t][b], u = res[t + (RS - R)][b];
                            out = (g / (1.0f + expf(-g))) * u;
                        } else {
                            out = res[t][b] * rms_inv[b];
                        }
                        p.y[(size_t)b * N + n] = __float2half_rn(out);
                    }
                }
            }
        }
    }
}

// Any group size / ragged K: one warp per row, plain float arithmetic.  Load-time and test
// shapes only; the decode shapes all take the streaming kernel above.
template <int MODE>
__global__ void matvec_generic_kernel(const MatvecParams p, int bits, int gs, int B) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= p.N) return;
    const int K = p.K, G = p.G;
    for (int b = 0; b < B; b++) {
        float acc0 = 0.0f, acc1 = 0.0f, sq = 0.0f;
        for (int k = lane; k < K; k += 32) {
            float xv = __half2float(p.x[(size_t)b * K + k]);
            if (MODE == kResidualNorm) {
                xv += __half2float(p.b[(size_t)b * K + k]);
                sq += xv * xv;
                xv *= __half2float(p.gamma[k]);
            }
            if (p.awq) xv = xv / __half2float(p.awq[k]);
            const size_t e = (size_t)n * K + k;
            auto deq = [&](const uint8_t *codes, const __half2 *sz) {
                unsigned q = bits == 4 ? ((codes[e >> 1] >> ((e & 1) * 4)) & 0xF) : codes[e];
                float2 s_z = __half22float2(sz[(size_t)n * G + k / gs]);
                return ((float)q - s_z.y) * s_z.x;
            };
            acc0 += xv * deq(p.codes0, p.sz0);
            if (MODE == kGateUpAct) acc1 += xv * deq(p.codes1, p.sz1);
        }
        acc0 = warp_sum(acc0);
        if (MODE == kGateUpAct) acc1 = warp_sum(acc1);
        float rms_inv = 1.0f;
        if (MODE == kResidualNorm) {
            sq = warp_sum(sq);
            rms_inv = rsqrtf(sq / (float)K + p.eps);
            if (n == 0)
                for (int k = lane; k < K; k += 32) {
                    float r = __half2float(p.x[(size_t)b * K + k]) + __half2float(p.b[(size_t)b * K + k]);
                    if (p.residual_out) p.residual_out[(size_t)b * K + k] = __float2half_rn(r);
                    if (p.normed_out) p.normed_out[(size_t)b * K + k] = __float2half_rn(r * rms_inv * __half2float(p.gamma[k]));
                }
        }
        if (lane == 0) {
            float out = MODE == kGateUpAct ? (acc0 / (1.0f + expf(-acc0))) * acc1 : acc0 * rms_inv;
            p.y[(size_t)b * p.N + n] = __float2half_rn(out);
        }
    }
}

// Dense fp16 matvec (lm_head): y[b,n] = sum_k W[n,k] x[b,k], f32 accumulation.
// crates/ironmill-inference/src/metal/shaders/linear/matvec.metal:30-84
template <int NB>
__global__ void __launch_bounds__(kThreads) matvec_f16_kernel(const __half *__restrict__ w, const __half *__restrict__ x,
                                                              __half *__restrict__ y, int N, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);  // [NB][K/8] blocks of 8 halves
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kb = K / 8;
    pdl_trigger();
    pdl_wait();
    for (int b = 0; b < NB; b++)
        for (int i = threadIdx.x; i < kb; i += kThreads) xs[b * kb + i] = reinterpret_cast<const uint4 *>(x + (size_t)b * K)[i];
    __syncthreads();
    constexpr int R = 2;
    const int ntiles = (N + kWarps * R - 1) / (kWarps * R);
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int n0 = (tile * kWarps + warp) * R;
        float acc[R][NB];
#pragma unroll
        for (int t = 0; t < R; t++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[t][b] = 0.0f;
#pragma unroll 4
        for (int i = lane; i < kb; i += 32) {
            uint4 wv[R];
#pragma unroll
            for (int t = 0; t < R; t++) wv[t] = ldg_stream_v4(w + (size_t)min(n0 + t, N - 1) * K + (size_t)i * 8);
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const uint4 xr = xs[b * kb + i];
                const __half2 *hx = reinterpret_cast<const __half2 *>(&xr);
                const float2 x0 = __half22float2(hx[0]), x1 = __half22float2(hx[1]), x2 = __half22float2(hx[2]), x3 = __half22float2(hx[3]);
#pragma unroll
                for (int t = 0; t < R; t++) {
                    const __half2 *h = reinterpret_cast<const __half2 *>(&wv[t]);
                    const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
                    float a = acc[t][b];
                    a = fmaf(f0.x, x0.x, a); a = fmaf(f0.y, x0.y, a); a = fmaf(f1.x, x1.x, a); a = fmaf(f1.y, x1.y, a);
                    a = fmaf(f2.x, x2.x, a); a = fmaf(f2.y, x2.y, a); a = fmaf(f3.x, x3.x, a); a = fmaf(f3.y, x3.y, a);
                    acc[t][b] = a;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < R; t++)
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float s = warp_sum(acc[t][b]);
                if (lane == 0 && n0 + t < N) y[(size_t)b * N + n0 + t] = __float2half_rn(s);
            }
    }
}

__global__ void matvec_f16_generic_kernel(const __half *__restrict__ w, const __half *__restrict__ x,
                                          __half *__restrict__ y, int N, int K, int B) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    for (int b = 0; b < B; b++) {
        float acc = 0.0f;
        for (int k = lane; k < K; k += 32) acc += __half2float(w[(size_t)n * K + k]) * __half2float(x[(size_t)b * K + k]);
        acc = warp_sum(acc);
        if (lane == 0) y[(size_t)b * N + n] = __float2half_rn(acc);
    }
}

// ---- load-time repack ------------------------------------------------------
// Scales / zero points (f32 or fp16 as stored in the bundle) -> fp16 RNE, interleaved (s, z).
__global__ void interleave_params_kernel(const void *scales, const void *zeros, int is_f32, size_t n, __half2 *out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    __half s, z;
    if (is_f32) {
        s = __float2half_rn(static_cast<const float *>(scales)[i]);
        z = __float2half_rn(static_cast<const float *>(zeros)[i]);
    } else {
        s = static_cast<const __half *>(scales)[i];
        z = static_cast<const __half *>(zeros)[i];
    }
    out[i] = __halves2half2(s, z);
}

__global__ void dequant_kernel(const uint8_t *codes, const __half2 *sz, int bits, int gs, int G, size_t N, size_t K, __half *out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * K) return;
    size_t n = i / K, k = i % K;
    unsigned q = bits == 4 ? ((codes[i >> 1] >> ((i & 1) * 4)) & 0xF) : codes[i];
    float2 s_z = __half22float2(sz[n * G + k / gs]);
    out[i] = __float2half_rn(__fmul_rn(__fsub_rn((float)q, s_z.y), s_z.x));
}

static bool fast_path(const AffineWeight *w) {
    return w->group_size == kGroup && w->K % kGroup == 0 && w->K >= kGroup;
}

template <int BITS, int MODE, int R, int NB>
static int launch_fast(const MatvecParams &p, const Device *dev, cudaStream_t st) {
    constexpr int kChunk = Lay<BITS>::kChunk, kXV = Lay<BITS>::kXV;
    constexpr int RS = MODE == kGateUpAct ? 2 * R : R;
    const int nchunks = (p.K + kChunk - 1) / kChunk;
    size_t smem = (size_t)NB * nchunks * (kXV * 32 * 16 + 32 * 8) + (size_t)(kWarps * RS * NB + kWarps + 1) * 4;
    if (smem > dev->smem_optin) return fail(IM_ERR_INVALID, "K=%d needs %zu bytes of shared memory per CTA (limit %zu)", p.K, smem, dev->smem_optin);
    auto kern = matvec_kernel<BITS, MODE, R, NB>;
    static DeviceOnce once;  // per instantiation
    if (smem > 48 * 1024 && once.first(dev->ordinal))
        IM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev->smem_optin));
    const int rows_per_tile = (kWarps / p.ksplit) * R;
    const int ntiles = (p.N + rows_per_tile - 1) / rows_per_tile;
    int ctas_per_sm = smem > 0 ? (int)((200 * 1024) / (smem + 1024)) : 8;
    ctas_per_sm = ctas_per_sm < 1 ? 1 : (ctas_per_sm > 4 ? 4 : ctas_per_sm);
    const int max_grid = dev->sm_count * ctas_per_sm;
    const int tiles_per_cta = (ntiles + max_grid - 1) / max_grid;
    const int grid = (ntiles + tiles_per_cta - 1) / tiles_per_cta;  // equal work per CTA
    kern<<<grid, kThreads, smem, st>>>(p);
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
}

// Pick how many warps split K: enough warp tasks to fill the machine for short matrices.
static int pick_ksplit(const Device *dev, int N, int K, int R, int chunk) {
    const int nchunks = (K + chunk - 1) / chunk;
    int ks = 1;
    const long want = (long)dev->sm_count * 16;
    while (ks < kWarps && ks * 2 <= nchunks && (long)((N + R - 1) / R) * ks < want) ks *= 2;
    return ks;
}


// Gate/up pair as one tile stream (8 gate rows + 8 up rows per tile), built the first time the pair is used.
int ensure_pair(const AffineWeight *gate_c, const AffineWeight *up, cudaStream_t st) {
    AffineWeight *gate = const_cast<AffineWeight *>(gate_c);
    if (gate->pair_with == up && gate->pair_tiles) return IM_OK;
    dev_free(gate->dev, gate->pair_tiles, (size_t)gate->pair_nblk * gate->G * 1088);
    gate->pair_tiles = nullptr;
    gate->pair_with = nullptr;
    gate->pair_nblk = (gate->N + 7) / 8;
    int rc = dev_malloc(gate->dev, (void **)&gate->pair_tiles, (size_t)gate->pair_nblk * gate->G * 1088);
    if (rc != IM_OK) return rc;
    gate->bytes += (size_t)gate->pair_nblk * gate->G * 1088;
    rc = v2_repack(gate->codes, gate->sz, up->codes, up->sz, gate->N, gate->K, gate->G, gate->pair_nblk, 8, gate->pair_tiles, st);
    if (rc == IM_OK) gate->pair_with = up;
    return rc;
}

template <int MODE>
static int run_matvec_v2(const MatvecParams &p, const AffineWeight *w, const AffineWeight *up, int B, cudaStream_t st) {
    V2Params q{};
    if (w->bits != 4 && MODE != kPlain) return IM_ERR_BOUNDS;  // 8-bit tiles: the plain projection only
    if (MODE & 1) {
        if ((w->N + 7) / 8 > kSkMaxBlocks) return IM_ERR_BOUNDS;
        int rc = ensure_pair(w, up, st);
        if (rc != IM_OK) return rc;
        q.tiles = w->pair_tiles;
        q.nblk = w->pair_nblk;
    } else {
        q.tiles = w->tiles;
        q.nblk = w->nblk;
    }
    q.awq = p.awq; q.gamma = p.gamma; q.eps = p.eps;
    q.N = p.N; q.K = p.K; q.G = p.G;
    q.partial = w->dev->sk_partial; q.counters = w->dev->sk_counters; q.err = w->dev->err_flag;
    int done = 0;
    while (done < B) {
        int nb = B - done >= 4 ? 4 : (B - done >= 2 ? 2 : 1);
        q.x = p.x + (size_t)done * p.K;
        q.b = p.b ? p.b + (size_t)done * p.K : nullptr;
        q.y = p.y + (size_t)done * p.N;
        q.residual_out = p.residual_out ? p.residual_out + (size_t)done * p.K : nullptr;
        q.normed_out = p.normed_out ? p.normed_out + (size_t)done * p.K : nullptr;
        int rc = v2_run(MODE, nb, q, w->dev, st, w->bits);
        // the staged activations of four (or two) batch rows may not fit beside the ring for a long K: fewer rows per launch
        while (rc == IM_ERR_BOUNDS && nb > 1) {
            nb /= 2;
            rc = v2_run(MODE, nb, q, w->dev, st, w->bits);
        }
        if (rc != IM_OK) return rc;  // IM_ERR_BOUNDS on the first chunk: caller falls back
        done += nb;
    }
    return IM_OK;
}

template <int MODE>
static int run_matvec(MatvecParams p, const AffineWeight *w, int B, cudaStream_t st, const AffineWeight *up = nullptr) {
    const Device *dev = w->dev;
    const size_t xstride = (size_t)p.K, ystride = (size_t)p.N;
    if (w->tiles && (w->bits == 4 || MODE == kPlain) && (MODE != kGateUpAct || (up && up->tiles && up->bits == 4))) {
        const int rc = run_matvec_v2<MODE>(p, w, up, B, st);
        if (rc != IM_ERR_BOUNDS) return rc;  // shapes whose activations do not fit beside the ring use the kernel below
    }
    if (!fast_path(w)) {
        const int wpb = 8;
        matvec_generic_kernel<MODE><<<(p.N + wpb - 1) / wpb, wpb * 32, 0, st>>>(p, w->bits, w->group_size, B);
        IM_CUDA_CHECK(cudaGetLastError());
        return IM_OK;
    }
    constexpr int R = MODE == kGateUpAct ? 2 : 4;
    int done = 0;
    while (done < B) {
        int nb = B - done >= 4 ? 4 : (B - done >= 2 ? 2 : 1);
        MatvecParams q = p;
        q.x = p.x + (size_t)done * xstride;
        if (p.b) q.b = p.b + (size_t)done * xstride;
        q.y = p.y + (size_t)done * ystride;
        if (p.residual_out) q.residual_out = p.residual_out + (size_t)done * xstride;
        if (p.normed_out) q.normed_out = p.normed_out + (size_t)done * xstride;
        int rc;
        if (w->bits == 4) {
            q.ksplit = pick_ksplit(dev, p.N, p.K, R, Lay<4>::kChunk);
            rc = nb == 4 ? launch_fast<4, MODE, R, 4>(q, dev, st) : nb == 2 ? launch_fast<4, MODE, R, 2>(q, dev, st) : launch_fast<4, MODE, R, 1>(q, dev, st);
        } else {
            q.ksplit = pick_ksplit(dev, p.N, p.K, R, Lay<8>::kChunk);
            rc = nb == 4 ? launch_fast<8, MODE, R, 4>(q, dev, st) : nb == 2 ? launch_fast<8, MODE, R, 2>(q, dev, st) : launch_fast<8, MODE, R, 1>(q, dev, st);
        }
        if (rc != IM_OK) return rc;
        done += nb;
    }
    return IM_OK;
}

static MatvecParams base_params(const AffineWeight *w) {
    MatvecParams p{};
    p.codes0 = w->codes;
    p.sz0 = w->sz;
    p.awq = w->awq;
    p.N = w->N;
    p.K = w->K;
    p.G = w->G;
    p.ksplit = 1;
    return p;
}

}  // namespace im

static int weight_create_common(im_device *dev, const void *qdata, const void *scales, const void *zeros,
                                int param_dtype, const void *awq, int N, int K, int group_size, int bit_width,
                                bool host_src, cudaStream_t st, im_affine_weight **out) {
    using namespace im;
    IM_REQUIRE(dev && out, "bad argument");
    *out = nullptr;
    IM_REQUIRE(qdata && scales && zeros, "NULL weight data");
    IM_REQUIRE(N > 0 && K > 0, "N and K must be positive (got %d x %d)", N, K);
    IM_REQUIRE(bit_width == 4 || bit_width == 8, "bit_width must be 4 or 8, got %d", bit_width);
    IM_REQUIRE(group_size > 0, "group_size must be positive");
    IM_REQUIRE(param_dtype == IM_DTYPE_F16 || param_dtype == IM_DTYPE_F32, "param_dtype must be IM_DTYPE_F16 or IM_DTYPE_F32");
    IM_CUDA_CHECK(cudaSetDevice(dev->ordinal));
    im_affine_weight *w = new im_affine_weight();
    w->dev = dev;
    w->N = N;
    w->K = K;
    w->group_size = group_size;
    w->bits = bit_width;
    w->G = (K + group_size - 1) / group_size;
    const size_t code_bytes = bit_width == 4 ? ((size_t)N * K + 1) / 2 : (size_t)N * K;
    const size_t nparams = (size_t)N * w->G;
    const size_t psz = param_dtype == IM_DTYPE_F32 ? 4 : 2;
    void *tmp_s = nullptr, *tmp_z = nullptr;
    int rc = IM_OK;
    auto cleanup = [&]() {
        cudaFree(tmp_s);
        cudaFree(tmp_z);
    };
    auto bail = [&](int code) {
        cleanup();
        im_cuda_affine_weight_free(w);
        return code;
    };
    const size_t code_alloc = (code_bytes + 15) / 16 * 16;
    if ((rc = dev_malloc(dev, (void **)&w->codes, code_alloc)) != IM_OK) return bail(rc);
    w->bytes += code_alloc;
    if ((rc = dev_malloc(dev, (void **)&w->sz, nparams * sizeof(__half2))) != IM_OK) return bail(rc);
    w->bytes += nparams * sizeof(__half2);
    if (awq) {
        if ((rc = dev_malloc(dev, (void **)&w->awq, (size_t)K * sizeof(__half))) != IM_OK) return bail(rc);
        w->bytes += (size_t)K * sizeof(__half);
    }
    const cudaMemcpyKind kind = host_src ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    const void *ds = scales, *dz = zeros;
    cudaError_t e = cudaSuccess;
    if (host_src) {
        if (cudaMalloc(&tmp_s, nparams * psz) != cudaSuccess || cudaMalloc(&tmp_z, nparams * psz) != cudaSuccess) {
            cudaGetLastError();
            return bail(fail(IM_ERR_ALLOC, "staging allocation failed"));
        }
        e = cudaMemcpyAsync(tmp_s, scales, nparams * psz, kind, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(tmp_z, zeros, nparams * psz, kind, st);
        ds = tmp_s;
        dz = tmp_z;
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->codes, qdata, code_bytes, kind, st);
    if (e == cudaSuccess && awq) e = cudaMemcpyAsync(w->awq, awq, (size_t)K * sizeof(__half), kind, st);
    if (e != cudaSuccess) return bail(fail(IM_ERR_CUDA, "weight copy failed: %s", cudaGetErrorString(e)));
    interleave_params_kernel<<<(unsigned)((nparams + 255) / 256), 256, 0, st>>>(ds, dz, param_dtype == IM_DTYPE_F32, nparams, w->sz);
    e = cudaGetLastError();
    if (e == cudaSuccess && host_src) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return bail(fail(IM_ERR_CUDA, "weight repack failed: %s", cudaGetErrorString(e)));
    cleanup();
    if ((bit_width == 4 || bit_width == 8) && group_size == kGroup && K % kGroup == 0 && (N + 15) / 16 <= kSkMaxBlocks) {
        // tile-major copy for the bulk-staged kernel
        w->nblk = (N + 15) / 16;
        const size_t tb = (size_t)w->nblk * w->G * tile_bytes_of(bit_width);
        if ((rc = dev_malloc(dev, (void **)&w->tiles, tb)) != IM_OK) return bail(rc);
        w->bytes += tb;
        rc = bit_width == 4 ? v2_repack(w->codes, w->sz, nullptr, nullptr, N, K, w->G, w->nblk, 16, w->tiles, st)
                            : v2_repack8(w->codes, w->sz, N, K, w->G, w->nblk, w->tiles, st);
        if (rc == IM_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(IM_ERR_CUDA, "tile repack failed");
        if (rc != IM_OK) return bail(rc);
    }
    *out = w;
    return IM_OK;
}

IM_EXPORT int im_cuda_affine_weight_create(im_device *dev, const void *qdata_host, const void *scales_host,
                                           const void *zeros_host, int param_dtype, const void *awq_f16_host,
                                           int N, int K, int group_size, int bit_width, im_affine_weight **out) {
    IM_GUARD_BEGIN
    return weight_create_common(dev, qdata_host, scales_host, zeros_host, param_dtype, awq_f16_host, N, K, group_size,
                                bit_width, true, nullptr, out);
    IM_GUARD_END
}

IM_EXPORT int im_cuda_affine_weight_create_dev(im_device *dev, const void *qdata_dev, const void *scales_dev,
                                               const void *zeros_dev, int param_dtype, const void *awq_f16_dev,
                                               int N, int K, int group_size, int bit_width, void *stream,
                                               im_affine_weight **out) {
    IM_GUARD_BEGIN
    return weight_create_common(dev, qdata_dev, scales_dev, zeros_dev, param_dtype, awq_f16_dev, N, K, group_size,
                                bit_width, false, im::as_stream(stream), out);
    IM_GUARD_END
}

IM_EXPORT void im_cuda_affine_weight_free(im_affine_weight *w) {
    if (!w) return;
    const size_t code_bytes = w->bits == 4 ? ((size_t)w->N * w->K + 1) / 2 : (size_t)w->N * w->K;
    im::dev_free(w->dev, w->codes, (code_bytes + 15) / 16 * 16);
    im::dev_free(w->dev, w->sz, (size_t)w->N * w->G * sizeof(__half2));
    im::dev_free(w->dev, w->awq, (size_t)w->K * sizeof(__half));
    im::dev_free(w->dev, w->tiles, (size_t)w->nblk * w->G * im::tile_bytes_of(w->bits));
    im::dev_free(w->dev, w->pair_tiles, (size_t)w->pair_nblk * w->G * 1088);
    delete w;
}

IM_EXPORT size_t im_cuda_affine_weight_bytes(const im_affine_weight *w) { return w ? w->bytes : 0; }

IM_EXPORT int im_cuda_affine_weight_dequant(const im_affine_weight *w, void *out_f16_dev, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(w && out_f16_dev, "bad argument");
    size_t total = (size_t)w->N * w->K;
    im::dequant_kernel<<<(unsigned)((total + 255) / 256), 256, 0, im::as_stream(stream)>>>(
        w->codes, w->sz, w->bits, w->group_size, w->G, w->N, w->K, static_cast<__half *>(out_f16_dev));
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_matvec_affine(const im_affine_weight *w, const void *x_dev, void *y_dev, int B, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(w && x_dev && y_dev, "bad argument");
    IM_REQUIRE(B >= 1 && B <= 64, "batch must be in 1..64, got %d", B);
    im::MatvecParams p = im::base_params(w);
    p.x = static_cast<const __half *>(x_dev);
    p.y = static_cast<__half *>(y_dev);
    return im::run_matvec<im::kPlain>(p, w, B, im::as_stream(stream));
    IM_GUARD_END
}

IM_EXPORT int im_cuda_matvec_affine_host(const im_affine_weight *w, const void *x_host, void *y_host, int B) {
    IM_GUARD_BEGIN
    IM_REQUIRE(w && x_host && y_host, "bad argument");
    IM_REQUIRE(B >= 1 && B <= 64, "batch must be in 1..64, got %d", B);
    IM_CUDA_CHECK(cudaSetDevice(w->dev->ordinal));
    const size_t xb = (size_t)B * w->K * 2, yb = (size_t)B * w->N * 2;
    void *xd = nullptr, *yd = nullptr;
    IM_CUDA_CHECK(cudaMalloc(&xd, xb));
    cudaError_t e = cudaMalloc(&yd, yb);
    int rc = IM_OK;
    if (e != cudaSuccess) rc = im::fail(IM_ERR_ALLOC, "cudaMalloc failed: %s", cudaGetErrorString(e));
    if (rc == IM_OK && (e = cudaMemcpy(xd, x_host, xb, cudaMemcpyHostToDevice)) != cudaSuccess)
        rc = im::fail(IM_ERR_CUDA, "copy in failed: %s", cudaGetErrorString(e));
    if (rc == IM_OK) rc = im_cuda_matvec_affine(w, xd, yd, B, nullptr);
    if (rc == IM_OK && (e = cudaMemcpy(y_host, yd, yb, cudaMemcpyDeviceToHost)) != cudaSuccess)
        rc = im::fail(IM_ERR_CUDA, "copy out failed: %s", cudaGetErrorString(e));
    cudaFree(xd);
    cudaFree(yd);
    return rc;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_ffn_gate_up_act(const im_affine_weight *gate, const im_affine_weight *up, const void *x_dev,
                                      void *out_dev, int B, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(gate && up && x_dev && out_dev, "bad argument");
    IM_REQUIRE(B >= 1 && B <= 64, "batch must be in 1..64, got %d", B);
    IM_REQUIRE(gate->N == up->N && gate->K == up->K && gate->bits == up->bits && gate->group_size == up->group_size,
               "gate [%d,%d] and up [%d,%d] must have the same shape and format", gate->N, gate->K, up->N, up->K);
    im::MatvecParams p = im::base_params(gate);
    p.codes1 = up->codes;
    p.sz1 = up->sz;
    p.x = static_cast<const __half *>(x_dev);
    p.y = static_cast<__half *>(out_dev);
    return im::run_matvec<im::kGateUpAct>(p, gate, B, im::as_stream(stream), up);
    IM_GUARD_END
}

IM_EXPORT int im_cuda_fused_residual_norm_matvec(const im_affine_weight *w, const void *a_dev, const void *b_dev,
                                                 const void *gamma_dev, float eps, void *y_dev,
                                                 void *residual_out_dev, void *normed_out_dev, int B, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(w && a_dev && b_dev && gamma_dev && y_dev, "bad argument");
    IM_REQUIRE(B >= 1 && B <= 64, "batch must be in 1..64, got %d", B);
    im::MatvecParams p = im::base_params(w);
    p.x = static_cast<const __half *>(a_dev);
    p.b = static_cast<const __half *>(b_dev);
    p.gamma = static_cast<const __half *>(gamma_dev);
    p.eps = eps;
    p.y = static_cast<__half *>(y_dev);
    p.residual_out = static_cast<__half *>(residual_out_dev);
    p.normed_out = static_cast<__half *>(normed_out_dev);
    return im::run_matvec<im::kResidualNorm>(p, w, B, im::as_stream(stream));
    IM_GUARD_END
}

IM_EXPORT int im_cuda_fused_residual_norm_ffn(const im_affine_weight *gate, const im_affine_weight *up, const void *a_dev,
                                              const void *b_dev, const void *gamma_dev, float eps, void *out_dev,
                                              void *residual_out_dev, void *normed_out_dev, int B, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(gate && up && a_dev && b_dev && gamma_dev && out_dev, "bad argument");
    IM_REQUIRE(B >= 1 && B <= 64, "batch must be in 1..64, got %d", B);
    IM_REQUIRE(gate->N == up->N && gate->K == up->K && gate->bits == up->bits && gate->group_size == up->group_size,
               "gate [%d,%d] and up [%d,%d] must have the same shape and format", gate->N, gate->K, up->N, up->K);
    cudaStream_t st = im::as_stream(stream);
    if (gate->tiles && up->tiles) {
        im::MatvecParams p = im::base_params(gate);
        p.x = static_cast<const __half *>(a_dev);
        p.b = static_cast<const __half *>(b_dev);
        p.gamma = static_cast<const __half *>(gamma_dev);
        p.eps = eps;
        p.y = static_cast<__half *>(out_dev);
        p.residual_out = static_cast<__half *>(residual_out_dev);
        p.normed_out = static_cast<__half *>(normed_out_dev);
        const int rc = im::run_matvec_v2<im::kResNormGateUp>(p, gate, up, B, st);
        if (rc != IM_ERR_BOUNDS) return rc;
    }
    // formats without the tiled layout: the two-step form
    IM_REQUIRE(residual_out_dev && normed_out_dev, "this weight format needs residual_out and normed_out buffers");
    int rc = im_cuda_fused_residual_rms_norm(a_dev, b_dev, gamma_dev, normed_out_dev, residual_out_dev, gate->K, B, eps, stream);
    if (rc != IM_OK) return rc;
    return im_cuda_ffn_gate_up_act(gate, up, normed_out_dev, out_dev, B, stream);
    IM_GUARD_END
}

IM_EXPORT int im_cuda_matvec_f16(const void *w_dev, const void *x_dev, void *y_dev, int N, int K, int B, void *stream) {
    IM_GUARD_BEGIN
    using namespace im;
    IM_REQUIRE(w_dev && x_dev && y_dev, "bad argument");
    IM_REQUIRE(N > 0 && K > 0, "N and K must be positive");
    IM_REQUIRE(B >= 1 && B <= 64, "batch must be in 1..64, got %d", B);
    cudaStream_t st = as_stream(stream);
    const __half *w = static_cast<const __half *>(w_dev);
    const __half *x = static_cast<const __half *>(x_dev);
    __half *y = static_cast<__half *>(y_dev);
    int devid = 0, sms = 0;
    IM_CUDA_CHECK(cudaGetDevice(&devid));
    IM_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, devid));
    if (K % 8 != 0 || (size_t)K * 2 * 4 > 160 * 1024) {
        matvec_f16_generic_kernel<<<(N + 7) / 8, 256, 0, st>>>(w, x, y, N, K, B);
        IM_CUDA_CHECK(cudaGetLastError());
        return IM_OK;
    }
    int done = 0;
    while (done < B) {
        const int nb = B - done >= 4 ? 4 : (B - done >= 2 ? 2 : 1);
        const size_t smem = (size_t)nb * K * 2;
        const int ntiles = (N + kWarps * 2 - 1) / (kWarps * 2);
        int cps = (int)((200 * 1024) / (smem + 1024));
        cps = cps < 1 ? 1 : (cps > 4 ? 4 : cps);
        int grid = sms * cps < ntiles ? sms * cps : ntiles;
        auto launch = [&](auto kern) -> int {
            if (smem > 48 * 1024) IM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            IM_CUDA_CHECK(launch_k(kern, dim3(grid), dim3(kThreads), smem, st, w, x + (size_t)done * K, y + (size_t)done * N, N, K));
            return IM_OK;
        };
        int rc = nb == 4 ? launch(matvec_f16_kernel<4>) : nb == 2 ? launch(matvec_f16_kernel<2>) : launch(matvec_f16_kernel<1>);
        if (rc != IM_OK) return rc;
        done += nb;
    }
    return IM_OK;
    IM_GUARD_END
}

// superblock_matmul_int4 (crates/ironmill-inference/src/metal/shaders/quantized/affine_matmul.metal:10-152) on the
// tcgen05 tensor cores (gemm_tc.cu).  INT4 group-128 weights only.
IM_EXPORT int im_cuda_matmul_affine(const im_affine_weight *w, const void *x_dev, void *y_dev, int M, void *scratch_dev, void *stream) {
    IM_GUARD_BEGIN
    using namespace im;
    IM_REQUIRE(w && x_dev && y_dev && scratch_dev, "bad argument");
    IM_REQUIRE(M >= 0, "M must be >= 0");
    if (M == 0) return IM_OK;
    IM_CUDA_CHECK(cudaSetDevice(w->dev->ordinal));
    const int rc = gemm_affine_tc(w, static_cast<const __half *>(x_dev), static_cast<__half *>(y_dev), M, static_cast<__half *>(scratch_dev),
                                  as_stream(stream));
    if (rc == IM_ERR_BOUNDS) return fail(IM_ERR_INVALID, "the tensor-core GEMM takes INT4 or INT8 group-128 weights with K a multiple of 128");
    return rc;
    IM_GUARD_END
}
