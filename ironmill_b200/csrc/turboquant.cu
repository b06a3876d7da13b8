// TurboQuant 8-bit KV cache: encoder and split-K decode attention.
//   constants   crates/ironmill-inference/src/turboquant/codebook.rs:20-200 (Lloyd-Max codebooks),
//               crates/ironmill-inference/src/turboquant/rotation.rs:13-49 (signs, QJL matrix),
//               crates/ironmill-inference/src/metal/turboquant/mod.rs:221-287
//   encode      crates/ironmill-inference/src/metal/shaders/turboquant/turboquant.metal:52-170
//               (turboquant_cache_write) + src/shaders/turboquant_helpers.metal:128-157
//   attention   .../turboquant/turboquant.metal:202-462 (turboquant_attention, split mode),
//               .../attention/flash_decode.metal:163-215 (fused_sdpa_reduce)
//
// Storage (per sequence): K and V caches [nkv, max_seq, hd] bytes, K = 7-bit codebook index |
// QJL sign in bit 7, V = 8-bit codebook index; f32 scale (L2 norm) per (head, position) for K
// and V and an f32 residual norm for K: 268 bytes per (kv head, position) at hd = 128.
//
// The encoder reproduces the reference arithmetic operation by operation (explicit
// round-to-nearest intrinsics, the same butterfly and tree-reduction order, sequential QJL dot
// product), so its bytes and norms are bit-identical to the CPU restatement.
// The attention kernel streams each K/V tile once per KV head for all query heads of its GQA
// group, splits the sequence across CTAs and combines the splits in a reduce kernel.
#include <math.h>

#include <new>
#include <vector>

#include "common.cuh"
#include "tq_device.cuh"

namespace im {

// ---------------------------------------------------------------- host: Lloyd-Max codebook
namespace lm {
static double poly(const double *c, int n, double x) {
    double r = c[0];
    for (int i = 1; i < n; i++) r = r * x + c[i];
    return r;
}
static double erf_as(double x) {  // codebook.rs:187-200
    static const double a[5] = {1.061405429, -1.453152027, 1.421413741, -0.284496736, 0.254829592};
    const double sign = x < 0.0 ? -1.0 : 1.0;
    x = fabs(x);
    const double t = 1.0 / (1.0 + 0.3275911 * x);
    const double y = 1.0 - (poly(a, 5, t) * t) * exp(-x * x);
    return sign * y;
}
static double pdf(double x) { return exp(-0.5 * x * x) / sqrt(2.0 * M_PI); }
static double cdf(double x) { return 0.5 * (1.0 + erf_as(x * M_SQRT1_2)); }
static double quantile(double p) {  // codebook.rs:114-184
    if (p <= 0.0) return -INFINITY;
    if (p >= 1.0) return INFINITY;
    const double t = p - 0.5;
    if (fabs(t) <= 0.42) {
        static const double n[4] = {2.5066282746310002, 18.6150006252966, 41.39119773534996, 25.44106049637689};
        static const double d[5] = {14.382029373388, 63.690613, 84.681, 40.304, 1.0};
        const double r = t * t;
        return t * poly(n, 4, r) / poly(d, 5, r);
    }
    const double r = t < 0.0 ? p : 1.0 - p;
    const double s = sqrt(-log(r));
    double v;
    if (s <= 5.0) {
        static const double n[8] = {0.000124818987, 0.0227061845, 0.2728688, 1.3058437, 2.7580128, 2.2311569, 0.6462025, 0.001612};
        static const double d[8] = {0.000038746, 0.00745102, 0.09234118, 0.4710441, 1.0507501, 1.0, 0.2127601, 1.0};
        v = poly(n, 8, s - 1.6) / poly(d, 8, s - 1.6);
    } else {
        static const double n[8] = {0.0000000271, 0.00000342556, 0.000170717, 0.004531901, 0.06871337, 0.56419917, 1.9715909, 2.1538256};
        static const double d[8] = {0.0000000393, 0.00000489649, 0.000230147, 0.005492439, 0.06353648, 0.3445453, 0.73741429, 1.0};
        v = poly(n, 8, s - 5.0) / poly(d, 8, s - 5.0);
    }
    return t < 0.0 ? -v : v;
}
static double cell_mean(double sigma, double lo, double hi) {  // codebook.rs:84-104
    const double lz = lo / sigma, hz = hi / sigma;
    const double prob = cdf(hz) - cdf(lz);
    if (prob < 1e-30) return isinf(lo) ? hi : (isinf(hi) ? lo : (lo + hi) / 2.0);
    return sigma * (pdf(lz) - pdf(hz)) / prob;
}
static void lloyd_max(int dim, int bits, std::vector<float> &levels, std::vector<float> &bounds) {  // codebook.rs:20-52
    const double sigma = 1.0 / sqrt((double)dim);
    const int n = 1 << bits;
    std::vector<double> lv(n), nl(n), bd(n > 1 ? n - 1 : 0);
    for (int i = 0; i < n; i++) lv[i] = sigma * quantile(((double)i + 0.5) / (double)n);
    for (int it = 0; it < 200; it++) {
        for (int i = 0; i + 1 < n; i++) bd[i] = (lv[i] + lv[i + 1]) / 2.0;
        double delta = 0.0;
        for (int i = 0; i < n; i++) {
            nl[i] = cell_mean(sigma, i == 0 ? -INFINITY : bd[i - 1], i == n - 1 ? INFINITY : bd[i]);
            delta = fmax(delta, fabs(lv[i] - nl[i]));
        }
        lv = nl;
        if (delta < 1e-10) break;
    }
    levels.resize(n);
    bounds.resize(n - 1);
    for (int i = 0; i < n; i++) levels[i] = (float)lv[i];
    for (int i = 0; i + 1 < n; i++) bounds[i] = (float)((lv[i] + lv[i + 1]) / 2.0);
}
}  // namespace lm

// ---------------------------------------------------------------- kernels: one CTA per work item
// (the bodies live in tq_device.cuh, shared with the whole-token decode kernel)

// grid (nseq*T, nkv), hd threads (tokens on x: a long prefill has more tokens than the y dimension holds).
template <int BITS>
__global__ void tq_encode_kernel(const __half *__restrict__ kv, const EncodeTables tb_in, uint8_t *__restrict__ cache,
                                 float *__restrict__ scale_buf, float *__restrict__ r_norms, int nkv, int hd, int max_seq, int base_pos,
                                 const int *__restrict__ pos_dev, int T) {
    extern __shared__ float sh[];
    const int d = threadIdx.x, h = blockIdx.y, st = blockIdx.x;
    const int seq = st / T, t = st % T;
    const int pos = (base_pos + (pos_dev ? pos_dev[seq] : 0) + t) % max_seq;
    const size_t row = ((size_t)seq * nkv + h) * max_seq + pos;
    const CtaScope sc{d, (int)blockDim.x};
    EncodeTables tb = tb_in;
    tb.bits = BITS;  // a constant here: the packing branch of the body folds away
    tq_encode_body(sc, __half2float(kv[((size_t)st * nkv + h) * hd + d]), tb, sh, hd, cache + row * tq_row_bytes(tb.bits, hd), scale_buf + row,
                   r_norms ? r_norms + row : nullptr);
}

// grid (nkv, nseq*T, splits), 128 threads.
template <int GQ, int BITS>
__global__ void __launch_bounds__(kAttnThreads) tq_attention_kernel(const AttnParams p_in) {
    AttnParams p = p_in;
    p.bits = BITS;  // a constant here: the cache-format branches of the body fold away
    __shared__ AttnSmem<GQ> sm;
    __shared__ float cbk[128];
    __shared__ float cbv[256];
    const int tid = threadIdx.x;
    const int kvh = blockIdx.x, st = blockIdx.y, split = blockIdx.z;
    pdl_trigger();
    pdl_wait();
    const int seq = st / p.T, t = st % p.T;
    // never past the end of the head's rows, whatever a device-side position says (the host can only check base_pos)
    const int seq_len = min(p.base_pos + (p.pos_dev ? p.pos_dev[cache_slot(p.slot_map, seq)] : 0) + t + 1, p.max_seq);
    const int chunk = (seq_len + p.splits - 1) / p.splits;
    const int r0 = split * chunk, r1 = min(r0 + chunk, seq_len);
    const int kl = 1 << (p.bits - 1), vl = 1 << p.bits;  // codebook sizes: K keeps one bit for the QJL sign
    cbk[tid] = tid < kl ? p.k_cb[tid] : 0.0f;
    cbv[tid] = tid < vl ? p.v_cb[tid] : 0.0f;
    cbv[tid + 128] = tid + 128 < vl ? p.v_cb[tid + 128] : 0.0f;
    __syncthreads();
    const CtaScope sc{tid, kAttnThreads};
    tq_attention_item<GQ>(sc, sm, cbk, cbv, p, kvh, st, split, r0, r1);
}

// One launch between the QKV projection and the attention: grid (nseq*T, nh + 2 nkv), hd = 128 threads.
// (Tried for prefill chunks: 16 tokens per CTA with the QJL matrix held in 64 KB of shared memory instead of 64 KB read
// from L2 per (token, head): three resident CTAs per SM do not hide the per-token chain of block barriers; 2048-token
// prefill 71 -> 81 ms.  Sixteen small CTAs per SM, as here, do.)
template <int BITS>
__global__ void __launch_bounds__(kHd) tq_qkv_prep_kernel(const PrepArgs a_in) {
    __shared__ float sh[3 * kHd + 4];
    PrepArgs a = a_in;
    a.ktab.bits = a.vtab.bits = BITS;
    pdl_trigger();
    pdl_wait();
    const CtaScope sc{(int)threadIdx.x, kHd};
    tq_prep_item(sc, a, sh, blockIdx.y, blockIdx.x);
}

// grid (nseq*T, nh), hd threads.
__global__ void __launch_bounds__(kHd) tq_reduce_kernel(const float *__restrict__ po, const float *__restrict__ pm,
                                                        const float *__restrict__ pl, const float *__restrict__ signs,
                                                        __half *__restrict__ out, int nh, int splits) {
    __shared__ float x[kHd];
    pdl_trigger();
    pdl_wait();
    const CtaScope sc{(int)threadIdx.x, kHd};
    tq_reduce_item(sc, x, po, pm, pl, signs, out, (size_t)blockIdx.x * nh + blockIdx.y, splits, splits);
}


// ---------------------------------------------------------------- tensor-core attention (GQ <= 4, rotated queries given)
// The split attention above spends its time in shared-memory gathers (one codebook lookup per cached byte, bank
// conflicts included) and f32 FMAs; at long context it reaches a few per cent of HBM bandwidth.  This kernel keeps
// the same arithmetic contract and partial format but
//   * every warp walks its own run of 32-position tiles: the K and V rows go from global memory straight into
//     registers (a lane owns 32-byte / 16-byte pieces of whole rows, all coalesced), no block barrier in the loop;
//   * the codebooks are shared-memory tables replicated once per lane (entry b of lane l at word 32 b + l): a
//     gather never meets a bank conflict.  K entries carry (centroid, QJL sign) as an fp16 pair, V entries the centroid;
//   * the dot products run on mma.sync m16n8k16 (fp16 operands, f32 accumulation): scores as
//     [16 positions x 16 dims] x [16 dims x 8] with columns 0-3 = the GQ rotated queries against the centroid
//     fragment and columns 4-7 = S q against the sign fragment; outputs as [16 dims x 16 positions] x
//     [16 positions x 8 heads].  The fragment <-> (dimension, position) assignment is chosen so that a fragment
//     register is built from bytes the lane already holds.
// The eight warps of a CTA take consecutive runs of one (KV head, token, split) and merge their results in shared
// memory, so the number of partials per head is the same as with the kernel above.
constexpr int kTcWarps = 8;
__device__ __forceinline__ void mma_f16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// table word of element `idx` of cache word w for this lane: bytes (BITS = 8, idx 0-3) or nibbles (BITS = 4, idx 0-7)
template <int BITS>
__device__ __forceinline__ unsigned lut_at(unsigned lane_base, unsigned w, int idx) {
    const unsigned b = BITS == 8 ? __byte_perm(w, 0, 0x4440 + idx) : ((w >> (4 * idx)) & 15u);
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(b * 128u + lane_base));
    return v;
}
__device__ __forceinline__ unsigned pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&h);
}

template <int GQ, int BITS>
__global__ void __launch_bounds__(kTcWarps * 32, 2) tq_attention_tc_kernel(const AttnParams p) {
    constexpr int kRowB = BITS == 4 ? kHd / 2 : kHd;  // bytes of a cached row
    extern __shared__ __align__(16) unsigned char tc_smem[];
    unsigned *lutk = reinterpret_cast<unsigned *>(tc_smem);        // [256][32]: (centroid, sign) fp16 pair
    unsigned *lutv = lutk + 256 * 32;                               // [256][32]: (centroid, 0)
    __half *pw = reinterpret_cast<__half *>(lutv + 256 * 32);       // [warps][4 heads][32 positions] softmax weights x v scale
    float *comb = reinterpret_cast<float *>(pw + kTcWarps * 4 * 32);  // [warps][4 heads][130]: o, m, l of each warp

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.x, st = blockIdx.y, split = blockIdx.z;
    pdl_trigger();
    {   // tables (constants): before the dependency wait
        const int b = tid;  // 256 threads, one stored value each (4-bit caches use the first 16 entries)
        constexpr int kSign = 1 << (BITS - 1), kVals = 1 << BITS;
        const __half2 ke = __floats2half2_rn(p.k_cb[b & (kSign - 1)], (b & kSign) ? 1.0f : -1.0f);
        const __half2 ve = __floats2half2_rn(p.v_cb[b & (kVals - 1)], 0.0f);
        const unsigned ku = *reinterpret_cast<const unsigned *>(&ke), vu = *reinterpret_cast<const unsigned *>(&ve);
        uint4 *dk = reinterpret_cast<uint4 *>(lutk + b * 32), *dv = reinterpret_cast<uint4 *>(lutv + b * 32);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            dk[i] = make_uint4(ku, ku, ku, ku);
            dv[i] = make_uint4(vu, vu, vu, vu);
        }
    }
    pdl_wait();
    __syncthreads();

    const int seq = st / p.T, tt = st % p.T;
    const int slot = cache_slot(p.slot_map, seq);
    const int seq_len = min(p.base_pos + (p.pos_dev ? p.pos_dev[slot] : 0) + tt + 1, p.max_seq);  // see tq_attention_kernel
    const int chunk = (seq_len + p.splits - 1) / p.splits;
    const int c0 = split * chunk, c1 = min(c0 + chunk, seq_len);
    // this warp's run: whole tiles of the split's range
    const int tiles = (max(c1 - c0, 0) + kTile - 1) / kTile, per = (tiles + kTcWarps - 1) / kTcWarps;
    const int r0 = c0 + warp * per * kTile, r1 = min(c1, r0 + per * kTile);
    const int h0 = kvh * GQ;
    const size_t head_base = ((size_t)slot * p.nkv + kvh) * p.max_seq;
    const unsigned lk = (unsigned)__cvta_generic_to_shared(lutk) + lane * 4u, lv = (unsigned)__cvta_generic_to_shared(lutv) + lane * 4u;

    // B fragments of the score products: lane (n = g, t) holds dims 32 t + 4 j + {0..3} of column n: the rotated query
    // of head n (n < GQ, against centroids) or S q of head n - 4 (4 <= n < 4 + GQ, against signs); zero otherwise
    // (one register set: a lane has either query or S q values; the other product of the pair gets zeros)
    unsigned bx[16];
#pragma unroll
    for (int i = 0; i < 16; i++) bx[i] = 0u;
    const bool is_c = g < 4;  // this lane's column belongs to the centroid product
    if (g < GQ || (g >= 4 && g < 4 + GQ)) {
        const float *src = p.qrot + ((size_t)st * p.nh + h0 + (g < 4 ? g : g - 4)) * 2 * kHd + (g < 4 ? 0 : kHd) + 32 * t;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float4 v = *reinterpret_cast<const float4 *>(src + 4 * j);
            bx[2 * j] = pack_h2(v.x, v.y);
            bx[2 * j + 1] = pack_h2(v.z, v.w);
        }
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};  // lanes t < 2: heads 2t, 2t + 1
    float o[8][4];                                                       // o[mb]: dims 16g + 2mb, +1 (rows) x heads 2t, 2t+1
#pragma unroll
    for (int i = 0; i < 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    __half *pwarp = pw + warp * 4 * 32;

    for (int ts = r0; ts < r1; ts += kTile) {
        const int nt = min(kTile, r1 - ts);
        // ---- K rows g, g+8, g+16, g+24 of the tile: dims 32t .. 32t+31 each (32 bytes, or 16 bytes of nibbles) ----
        uint4 kq[4][BITS == 8 ? 2 : 1];
        float ksv[4], rwv[4], vsv[4];
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int pos = g + 8 * r;
            kq[r][0] = make_uint4(0, 0, 0, 0);
            if (BITS == 8) kq[r][BITS == 8 ? 1 : 0] = make_uint4(0, 0, 0, 0);
            ksv[r] = rwv[r] = vsv[r] = 0.0f;
            if (pos < nt) {
                const uint4 *src = reinterpret_cast<const uint4 *>(p.kc + (head_base + ts + pos) * kRowB + (kRowB / 4) * t);
                kq[r][0] = ldg_stream_v4(src);
                if (BITS == 8) kq[r][BITS == 8 ? 1 : 0] = ldg_stream_v4(src + 1);
                ksv[r] = p.ks[head_base + ts + pos];
                rwv[r] = p.krn[head_base + ts + pos] * p.qjl_factor;
                vsv[r] = p.vs[head_base + ts + pos];
            }
        }
        // ---- scores: two 16-position row blocks ----
        float sc[2][4];  // [row block][c0..c3]
#pragma unroll
        for (int rb = 0; rb < 2; rb++) {
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const unsigned *wa = reinterpret_cast<const unsigned *>(&kq[2 * rb][0]);      // row g + 16 rb
            const unsigned *wb = reinterpret_cast<const unsigned *>(&kq[2 * rb + 1][0]);  // row g + 8 + 16 rb
#pragma unroll
            for (int j = 0; j < 8; j++) {  // dims 32 t + 4 j + {0..3}: word j (bytes), or half of word j / 2 (nibbles)
                const unsigned a = BITS == 8 ? wa[j] : wa[j >> 1], b = BITS == 8 ? wb[j] : wb[j >> 1];
                constexpr int e1 = 1, e2 = 2, e3 = 3;
                const int e0 = BITS == 8 ? 0 : (j & 1) * 4;
                const unsigned la0 = lut_at<BITS>(lk, a, e0), la1 = lut_at<BITS>(lk, a, e0 + e1), la2 = lut_at<BITS>(lk, a, e0 + e2), la3 = lut_at<BITS>(lk, a, e0 + e3);
                const unsigned lb0 = lut_at<BITS>(lk, b, e0), lb1 = lut_at<BITS>(lk, b, e0 + e1), lb2 = lut_at<BITS>(lk, b, e0 + e2), lb3 = lut_at<BITS>(lk, b, e0 + e3);
                // centroids in the low halves, signs in the high halves
                mma_f16(c, __byte_perm(la0, la1, 0x5410), __byte_perm(lb0, lb1, 0x5410), __byte_perm(la2, la3, 0x5410),
                        __byte_perm(lb2, lb3, 0x5410), is_c ? bx[2 * j] : 0u, is_c ? bx[2 * j + 1] : 0u);
                mma_f16(c, __byte_perm(la0, la1, 0x7632), __byte_perm(lb0, lb1, 0x7632), __byte_perm(la2, la3, 0x7632),
                        __byte_perm(lb2, lb3, 0x7632), is_c ? 0u : bx[2 * j], is_c ? 0u : bx[2 * j + 1]);
            }
            sc[rb][0] = c[0]; sc[rb][1] = c[1]; sc[rb][2] = c[2]; sc[rb][3] = c[3];
        }
        // ---- V rows 2t, 2t+1, 2t+8, 2t+9 (+16): dims 16g .. 16g+15 each (16 bytes, or 8 bytes of nibbles in .x/.y) ----
        uint4 vq[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const int pos = 2 * t + (r & 1) + 8 * ((r >> 1) & 1) + 16 * (r >> 2);
            vq[r] = make_uint4(0, 0, 0, 0);
            if (pos < nt) {
                if (BITS == 8) {
                    vq[r] = ldg_stream_v4(reinterpret_cast<const uint4 *>(p.vc + (head_base + ts + pos) * kRowB + 16 * g));
                } else {
                    const uint2 v2 = __ldcs(reinterpret_cast<const uint2 *>(p.vc + (head_base + ts + pos) * kRowB + 8 * g));
                    vq[r].x = v2.x;
                    vq[r].y = v2.y;
                }
            }
        }

        // lanes t < 2 hold the centroid sums of heads 2t, 2t+1; lanes t + 2 the sign sums of the same heads
        float s[4][2];  // [position g + 8 r][head 2t + i]
#pragma unroll
        for (int rb = 0; rb < 2; rb++)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float other = __shfl_xor_sync(0xffffffffu, sc[rb][q], 2);
                const int r = 2 * rb + (q >> 1), i = q & 1;  // c0,c1: row g ; c2,c3: row g + 8
                const bool live = t < 2 && g + 8 * r < nt;  // lanes t >= 2 only feed the shuffle above
                s[r][i] = live ? p.attn_scale * (ksv[r] * (sc[rb][q] + rwv[r] * other)) : -INFINITY;
            }
        // ---- online softmax over the tile (meaningful on lanes t < 2; the others carry copies of no use) ----
        float wgt[4][2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float mx = fmaxf(fmaxf(s[0][i], s[1][i]), fmaxf(s[2][i], s[3][i]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[i], mx);
            const float corr = m_new == -INFINITY ? 1.0f : __expf(m_run[i] - m_new);
            float sum = 0.0f;
#pragma unroll
            for (int r = 0; r < 4; r++) {
                wgt[r][i] = s[r][i] == -INFINITY ? 0.0f : __expf(s[r][i] - m_new);
                sum += wgt[r][i];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            sum += __shfl_xor_sync(0xffffffffu, sum, 8);
            sum += __shfl_xor_sync(0xffffffffu, sum, 16);
            l_run[i] = l_run[i] * corr + sum;
            m_run[i] = m_new;
#pragma unroll
            for (int mb = 0; mb < 8; mb++) {  // heads 2t + i live in accumulator columns i (rows d0) and i + 2 (rows d1)
                o[mb][i] *= corr;
                o[mb][i + 2] *= corr;
            }
        }
        // weights x V scale, as fp16, to this warp's P[head][position] for the output products
        __syncwarp();
        if (t < 2) {
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int i = 0; i < 2; i++)
                    if (2 * t + i < 4) pwarp[(2 * t + i) * 32 + g + 8 * r] = __float2half_rn(wgt[r][i] * vsv[r]);
        }
        __syncwarp();
        // ---- outputs: O^T[dims][heads] += V^T[dims][positions] P^T[positions][heads] ----
#pragma unroll
        for (int kb = 0; kb < 2; kb++) {
            unsigned b0 = 0u, b1 = 0u;  // lane (n = g): P[head g][16 kb + 2t, +1] and [.. + 8, + 9]
            if (g < GQ) {
                b0 = *reinterpret_cast<const unsigned *>(pwarp + g * 32 + 16 * kb + 2 * t);
                b1 = *reinterpret_cast<const unsigned *>(pwarp + g * 32 + 16 * kb + 2 * t + 8);
            }
            const unsigned *v0 = reinterpret_cast<const unsigned *>(&vq[4 * kb + 0]);  // position 16 kb + 2t
            const unsigned *v1 = reinterpret_cast<const unsigned *>(&vq[4 * kb + 1]);  // + 1
            const unsigned *v2 = reinterpret_cast<const unsigned *>(&vq[4 * kb + 2]);  // + 8
            const unsigned *v3 = reinterpret_cast<const unsigned *>(&vq[4 * kb + 3]);  // + 9
#pragma unroll
            for (int mb = 0; mb < 8; mb++) {  // rows g, g + 8 of the block: dims 16 g + 2 mb, + 1
                const int w = BITS == 8 ? mb >> 1 : mb >> 2, by = BITS == 8 ? 2 * (mb & 1) : 2 * (mb & 3);
                const unsigned e00 = lut_at<BITS>(lv, v0[w], by), e01 = lut_at<BITS>(lv, v1[w], by), e10 = lut_at<BITS>(lv, v0[w], by + 1), e11 = lut_at<BITS>(lv, v1[w], by + 1);
                const unsigned f00 = lut_at<BITS>(lv, v2[w], by), f01 = lut_at<BITS>(lv, v3[w], by), f10 = lut_at<BITS>(lv, v2[w], by + 1), f11 = lut_at<BITS>(lv, v3[w], by + 1);
                mma_f16(o[mb], __byte_perm(e00, e01, 0x5410), __byte_perm(e10, e11, 0x5410), __byte_perm(f00, f01, 0x5410),
                        __byte_perm(f10, f11, 0x5410), b0, b1);
            }
        }
        __syncwarp();
    }

    // ---- merge the warps: comb[warp][head][130] = o (dims 0..127), m, l ----
    if (t < 2) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int h = 2 * t + i;
            if (h < 4) {
                float *dst = comb + (warp * 4 + h) * 130;
#pragma unroll
                for (int mb = 0; mb < 8; mb++) {
                    dst[16 * g + 2 * mb] = o[mb][i];
                    dst[16 * g + 2 * mb + 1] = o[mb][i + 2];
                }
                if (g == 0) {
                    dst[128] = m_run[i];
                    dst[129] = l_run[i];
                }
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < GQ * kHd; idx += kTcWarps * 32) {
        const int h = idx >> 7, d = idx & 127;
        float gm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kTcWarps; w++) gm = fmaxf(gm, comb[(w * 4 + h) * 130 + 128]);
        float acc = 0.0f, lsum = 0.0f;
#pragma unroll
        for (int w = 0; w < kTcWarps; w++) {
            const float m = comb[(w * 4 + h) * 130 + 128];
            const float corr = m == -INFINITY ? 0.0f : __expf(m - gm);
            acc += comb[(w * 4 + h) * 130 + d] * corr;
            lsum += comb[(w * 4 + h) * 130 + 129] * corr;
        }
        const size_t pi = ((size_t)st * p.nh + h0 + h) * p.splits + split;
        p.po[pi * kHd + d] = acc;
        if (d == 0) {
            p.pm[pi] = gm;
            p.pl[pi] = lsum;
        }
    }
}
constexpr size_t kTcSmem = 2 * 256 * 32 * 4 + kTcWarps * 4 * 32 * 2 + kTcWarps * 4 * 130 * 4;

// Rotated query and S * rotated query for every (token, head), computed once instead of once per split:
// grid (nseq*T, nh), 128 threads.  q fp16 [nseq*T, nh, 128] -> qrot f32 [nseq*T, nh, 2, 128].
__global__ void __launch_bounds__(kHd) tq_qrot_kernel(const __half *__restrict__ q, const float *__restrict__ signs,
                                                      const float *__restrict__ qjl_t, float *__restrict__ qrot, int nh) {
    __shared__ float sh[2 * kHd];
    pdl_trigger();
    pdl_wait();
    const int d = threadIdx.x;
    const size_t hi = (size_t)blockIdx.x * nh + blockIdx.y;
    const CtaScope sc{d, kHd};
    const float rq = hadamard_thread(sc, __half2float(q[hi * kHd + d]), signs[d], sh + kHd, kHd);
    sh[d] = rq;
    __syncthreads();
    float acc = 0.0f;
    for (int k0 = 0; k0 < kHd; k0 += 64) {
        float sv[64];
#pragma unroll
        for (int j = 0; j < 64; j++) sv[j] = qjl_t[(size_t)(k0 + j) * kHd + d];
#pragma unroll
        for (int j = 0; j < 64; j++) acc = fmaf(sv[j], sh[k0 + j], acc);
    }
    qrot[hi * 2 * kHd + d] = rq;
    qrot[hi * 2 * kHd + kHd + d] = acc;
}

}  // namespace im

using namespace im;
struct im_tq : im::Tq {};

IM_EXPORT int im_cuda_tq_lloyd_max(int dim, int n_bits, float *levels_out_host, float *bounds_out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(dim > 0 && n_bits >= 1 && n_bits <= 8 && levels_out_host && bounds_out_host, "bad argument");
    std::vector<float> lv, bd;
    lm::lloyd_max(dim, n_bits, lv, bd);
    for (size_t i = 0; i < lv.size(); i++) levels_out_host[i] = lv[i];
    for (size_t i = 0; i < bd.size(); i++) bounds_out_host[i] = bd[i];
    return IM_OK;
    IM_GUARD_END
}

// Seeded stand-in for the reference's StdRng draws (rotation.rs:13-49): a +-1 sign vector and an
// N(0,1) matrix by Box-Muller over a splitmix64 stream.  Any such pair is algorithmically valid;
// the reference's own values depend on the `rand` crate's generator.
IM_EXPORT int im_cuda_tq_generate(int head_dim, uint64_t seed, float *signs_out_host, float *qjl_out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(head_dim > 0 && signs_out_host && qjl_out_host, "bad argument");
    auto next = [](uint64_t &s) {
        s += 0x9E3779B97F4A7C15ull;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    };
    uint64_t s1 = seed;
    for (int i = 0; i < head_dim; i++) signs_out_host[i] = (next(s1) >> 63) ? 1.0f : -1.0f;
    uint64_t s2 = seed + 1;
    const size_t n = (size_t)head_dim * head_dim;
    for (size_t i = 0; i < n;) {
        double u1 = (double)(next(s2) >> 11) * (1.0 / 9007199254740992.0);
        const double u2 = (double)(next(s2) >> 11) * (1.0 / 9007199254740992.0);
        if (u1 < 1e-300) u1 = 1e-300;
        const double r = sqrt(-2.0 * log(u1)), th = 2.0 * M_PI * u2;
        qjl_out_host[i++] = (float)(r * cos(th));
        if (i < n) qjl_out_host[i++] = (float)(r * sin(th));
    }
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT void im_cuda_tq_free(im_tq *tq) {
    if (!tq) return;
    const size_t hd = tq->hd;
    dev_free(tq->dev, tq->signs, hd * 4);
    dev_free(tq->dev, tq->qjl, hd * hd * 4);
    dev_free(tq->dev, tq->qjl_t, hd * hd * 4);
    dev_free(tq->dev, tq->k_cb, (size_t)tq->k_levels * 4);
    dev_free(tq->dev, tq->k_bd, (size_t)tq->k_levels * 4);
    dev_free(tq->dev, tq->v_cb, (size_t)tq->v_levels * 4);
    dev_free(tq->dev, tq->v_bd, (size_t)tq->v_levels * 4);
    dev_free(tq->dev, tq->scratch, tq->scratch_bytes);
    delete tq;
}

IM_EXPORT int im_cuda_tq_create(im_device *dev, int head_dim, int n_bits, const float *signs_host, const float *qjl_host,
                                const float *k_levels_host, const float *k_bounds_host, const float *v_levels_host,
                                const float *v_bounds_host, im_tq **out) {
    IM_GUARD_BEGIN
    IM_REQUIRE(dev && out, "bad argument");
    *out = nullptr;
    IM_REQUIRE(n_bits == 8 || n_bits == 4, "n_bits must be 4 or 8, got %d", n_bits);
    IM_REQUIRE(head_dim >= 32 && head_dim <= 1024 && (head_dim & (head_dim - 1)) == 0, "head_dim must be a power of two in 32..1024");
    IM_REQUIRE(signs_host && qjl_host, "signs and QJL matrix are required");
    IM_CUDA_CHECK(cudaSetDevice(dev->ordinal));
    std::vector<float> kl, kb, vl, vb;
    if (!k_levels_host || !k_bounds_host) {
        lm::lloyd_max(head_dim, n_bits - 1, kl, kb);
        k_levels_host = kl.data();
        k_bounds_host = kb.data();
    }
    if (!v_levels_host || !v_bounds_host) {
        lm::lloyd_max(head_dim, n_bits, vl, vb);
        v_levels_host = vl.data();
        v_bounds_host = vb.data();
    }
    // suffix minima of the boundary tables (see tq_encode_kernel)
    std::vector<float> ksm(k_bounds_host, k_bounds_host + (1 << (n_bits - 1)) - 1), vsm(v_bounds_host, v_bounds_host + (1 << n_bits) - 1);
    for (int i = (int)ksm.size() - 2; i >= 0; i--) ksm[i] = fminf(ksm[i], ksm[i + 1]);
    for (int i = (int)vsm.size() - 2; i >= 0; i--) vsm[i] = fminf(vsm[i], vsm[i + 1]);
    k_bounds_host = ksm.data();
    v_bounds_host = vsm.data();
    im_tq *tq = new im_tq();
    tq->dev = dev;
    tq->hd = head_dim;
    tq->n_bits = n_bits;
    tq->k_levels = 1 << (n_bits - 1);
    tq->v_levels = 1 << n_bits;
    const size_t hd = head_dim;
    const size_t hd_sz = head_dim;
    std::vector<float> qt(hd_sz * hd_sz);
    for (size_t r = 0; r < hd_sz; r++)
        for (size_t c2 = 0; c2 < hd_sz; c2++) qt[c2 * hd_sz + r] = qjl_host[r * hd_sz + c2];
    struct Up { float **dst; const float *src; size_t n, alloc; };
    Up ups[] = {{&tq->signs, signs_host, hd, hd}, {&tq->qjl, qjl_host, hd * hd, hd * hd}, {&tq->qjl_t, qt.data(), hd * hd, hd * hd},
                {&tq->k_cb, k_levels_host, (size_t)tq->k_levels, (size_t)tq->k_levels},
                {&tq->k_bd, k_bounds_host, (size_t)tq->k_levels - 1, (size_t)tq->k_levels},
                {&tq->v_cb, v_levels_host, (size_t)tq->v_levels, (size_t)tq->v_levels},
                {&tq->v_bd, v_bounds_host, (size_t)tq->v_levels - 1, (size_t)tq->v_levels}};
    for (auto &u : ups) {
        int rc = dev_malloc(dev, (void **)u.dst, u.alloc * 4);
        if (rc == IM_OK && cudaMemcpy(*u.dst, u.src, u.n * 4, cudaMemcpyHostToDevice) != cudaSuccess)
            rc = fail(IM_ERR_CUDA, "constant upload failed");
        if (rc != IM_OK) {
            im_cuda_tq_free(tq);
            return rc;
        }
        tq->const_bytes += u.alloc * 4;
    }
    *out = tq;
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_tq_encode(const im_tq *tq, const void *kv_dev, int is_k, void *cache_dev, float *scale_dev, float *r_norms_dev,
                                int nseq, int nkv, int max_seq, int base_pos, const int *pos_dev, int T, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(tq && kv_dev && cache_dev && scale_dev, "bad argument");
    IM_REQUIRE(!is_k || r_norms_dev, "the K cache needs a residual-norm buffer");
    IM_REQUIRE(nseq >= 0 && nkv > 0 && max_seq > 0 && base_pos >= 0 && T >= 0, "bad shape");
    if (nseq == 0 || T == 0) return IM_OK;
    dim3 grid(nseq * T, nkv);
    const int hd = tq->hd;
    EncodeTables tb{tq->signs, is_k ? tq->k_cb : tq->v_cb, is_k ? tq->k_bd : tq->v_bd, tq->qjl_t, is_k ? tq->k_levels : tq->v_levels, is_k, tq->n_bits};
    auto kern = tq->n_bits == 4 ? tq_encode_kernel<4> : tq_encode_kernel<8>;
    kern<<<grid, hd, 3 * hd * sizeof(float), as_stream(stream)>>>(
        static_cast<const __half *>(kv_dev), tb, static_cast<uint8_t *>(cache_dev), scale_dev, r_norms_dev, nkv, hd, max_seq, base_pos, pos_dev, T);
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
    IM_GUARD_END
}

static size_t tq_partial_bytes(int nseq, int T, int nh, int head_dim, int splits) {
    return (size_t)nseq * T * nh * splits * (head_dim + 2) * sizeof(float);
}
// split partials, then the rotated queries of im_cuda_tq_attention's pre-pass
IM_EXPORT size_t im_cuda_tq_scratch_bytes(int nseq, int T, int nh, int head_dim, int splits) {
    return tq_partial_bytes(nseq, T, nh, head_dim, splits) + (size_t)nseq * T * nh * 2 * head_dim * sizeof(float);
}

IM_EXPORT int im_cuda_tq_reserve_scratch(im_tq *tq, size_t bytes) {
    IM_GUARD_BEGIN
    IM_REQUIRE(tq, "bad argument");
    if (bytes <= tq->scratch_bytes) return IM_OK;
    IM_CUDA_CHECK(cudaSetDevice(tq->dev->ordinal));
    IM_CUDA_CHECK(cudaDeviceSynchronize());  // earlier launches may still use the old buffer
    dev_free(tq->dev, tq->scratch, tq->scratch_bytes);
    tq->scratch = nullptr;
    tq->scratch_bytes = 0;
    int rc = dev_malloc(tq->dev, (void **)&tq->scratch, bytes);
    if (rc != IM_OK) return rc;
    tq->scratch_bytes = bytes;
    return IM_OK;
    IM_GUARD_END
}

namespace im {
int tq_prep_launch(const Tq *tq, const TqPrep &a, cudaStream_t st) {
    if (tq->hd != kHd) return fail(IM_ERR_INVALID, "the fused cache-write kernel is built for head_dim 128 (got %d)", tq->hd);
    if (a.nseq == 0 || a.T == 0) return IM_OK;
    PrepArgs k{};
    k.qkv = a.qkv; k.stride = a.stride; k.k_off = a.k_off; k.v_off = a.v_off; k.kv = a.kv; k.kv_stride = a.kv_stride;
    k.qw = a.qw; k.kw = a.kw; k.cosc = a.cosc; k.sinc = a.sinc;
    k.nh = a.nh; k.nkv = a.nkv; k.rotary_dim = a.rotary_dim ? a.rotary_dim : kHd; k.with_norm = a.with_norm;
    k.T = a.T; k.max_seq = a.max_seq; k.base_pos = a.base_pos; k.eps = a.eps; k.pos_dev = a.pos_dev; k.slot_map = a.slot_map;
    k.qrot = a.qrot; k.q_out = a.q_out; k.no_q_proj = a.no_q_proj;
    k.ktab = EncodeTables{tq->signs, tq->k_cb, tq->k_bd, tq->qjl_t, tq->k_levels, 1, tq->n_bits};
    k.vtab = EncodeTables{tq->signs, tq->v_cb, tq->v_bd, tq->qjl_t, tq->v_levels, 0, tq->n_bits};
    k.kc = a.kc; k.vc = a.vc; k.ks = a.ks; k.vs = a.vs; k.krn = a.krn;
    const int tokens = a.nseq * a.T;
    dim3 grid(tokens, a.nh + 2 * a.nkv);
    IM_CUDA_CHECK(launch_k(tq->n_bits == 4 ? tq_qkv_prep_kernel<4> : tq_qkv_prep_kernel<8>, grid, dim3(kHd), 0, st, k));
    return IM_OK;
}

// Combination of split partials (normalise, rotate back, fp16) for `tokens` x nh heads: shared with tq_prefill.cu.
int tq_reduce_launch(const Tq *tq, const float *po, const float *pm, const float *pl, __half *out, int tokens, int nh, int splits, cudaStream_t st) {
    IM_CUDA_CHECK(launch_k(tq_reduce_kernel, dim3(tokens, nh), dim3(kHd), 0, st, po, pm, pl, (const float *)tq->signs, out, nh, splits));
    return IM_OK;
}

int tq_auto_splits(const Device *dev, int nseq, int T, int nkv, int seq_len) {
    const int ctas = nseq * T * nkv;
    int s = (2 * dev->sm_count + ctas - 1) / ctas;                // two 8-warp CTAs per SM
    const int by_len = (seq_len + 8 * kTile - 1) / (8 * kTile);  // at least one tile per warp of a split
    if (s > by_len) s = by_len;
    if (s > 128) s = 128;
    return s < 1 ? 1 : s;
}

int tq_attention_launch(const Tq *tq, float *scratch, const __half *q, const uint8_t *kc, const uint8_t *vc, const float *ks,
                        const float *vs, const float *krn, float attn_scale, __half *out, int nseq, int nh, int nkv, int max_seq,
                        int base_pos, const int *pos_dev, int T, int splits, cudaStream_t st, const float *qrot, const int *slot_map) {
    AttnParams p{};
    p.qrot = qrot;
    p.slot_map = slot_map;
    p.bits = tq->n_bits;
    p.q = q; p.kc = kc; p.vc = vc; p.ks = ks; p.vs = vs; p.krn = krn;
    p.signs = tq->signs; p.qjl = tq->qjl_t; p.k_cb = tq->k_cb; p.v_cb = tq->v_cb;
    const size_t rows = (size_t)nseq * T * nh * splits;
    p.po = scratch;
    p.pm = scratch + rows * kHd;
    p.pl = p.pm + rows;
    p.attn_scale = attn_scale;
    p.qjl_factor = sqrtf(2.0f / 3.14159265f) / (float)tq->hd;
    p.nh = nh; p.nkv = nkv; p.max_seq = max_seq; p.base_pos = base_pos; p.T = T; p.splits = splits; p.pos_dev = pos_dev;
    if ((long long)nseq * T > 65535) return fail(IM_ERR_BOUNDS, "attention takes at most 65535 (sequence, token) pairs per call, got %lld", (long long)nseq * T);
    dim3 grid(nkv, nseq * T, splits);
    const int gq = nh / nkv;
    if (qrot && (gq == 1 || gq == 2 || gq == 4) && nh % nkv == 0) {  // tensor-core kernel (needs the rotated queries)
        static DeviceOnce once;
        if (once.first(tq->dev->ordinal)) {  // the instantiations share one function-pointer type: set them all once
            IM_CUDA_CHECK(cudaFuncSetAttribute(tq_attention_tc_kernel<1, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
            IM_CUDA_CHECK(cudaFuncSetAttribute(tq_attention_tc_kernel<2, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
            IM_CUDA_CHECK(cudaFuncSetAttribute(tq_attention_tc_kernel<4, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
            IM_CUDA_CHECK(cudaFuncSetAttribute(tq_attention_tc_kernel<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
            IM_CUDA_CHECK(cudaFuncSetAttribute(tq_attention_tc_kernel<2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
            IM_CUDA_CHECK(cudaFuncSetAttribute(tq_attention_tc_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
        }
        auto kern = tq->n_bits == 4 ? (gq == 1 ? tq_attention_tc_kernel<1, 4> : (gq == 2 ? tq_attention_tc_kernel<2, 4> : tq_attention_tc_kernel<4, 4>))
                                    : (gq == 1 ? tq_attention_tc_kernel<1, 8> : (gq == 2 ? tq_attention_tc_kernel<2, 8> : tq_attention_tc_kernel<4, 8>));
        int rc = IM_OK;
        IM_CUDA_CHECK(launch_k(kern, grid, dim3(kTcWarps * 32), kTcSmem, st, p));
        if (rc != IM_OK) return rc;
    } else
    {
        const bool b4 = tq->n_bits == 4;
        switch (nh / nkv) {
            case 1: IM_CUDA_CHECK(launch_k(b4 ? tq_attention_kernel<1, 4> : tq_attention_kernel<1, 8>, grid, dim3(kAttnThreads), 0, st, p)); break;
            case 2: IM_CUDA_CHECK(launch_k(b4 ? tq_attention_kernel<2, 4> : tq_attention_kernel<2, 8>, grid, dim3(kAttnThreads), 0, st, p)); break;
            case 4: IM_CUDA_CHECK(launch_k(b4 ? tq_attention_kernel<4, 4> : tq_attention_kernel<4, 8>, grid, dim3(kAttnThreads), 0, st, p)); break;
            case 8: IM_CUDA_CHECK(launch_k(b4 ? tq_attention_kernel<8, 4> : tq_attention_kernel<8, 8>, grid, dim3(kAttnThreads), 0, st, p)); break;
            default: return fail(IM_ERR_INVALID, "query heads per KV head must be 1, 2, 4 or 8 (got %d/%d)", nh, nkv);
        }
    }
    dim3 rgrid(nseq * T, nh);
    IM_CUDA_CHECK(launch_k(tq_reduce_kernel, rgrid, dim3(kHd), 0, st, (const float *)p.po, (const float *)p.pm, (const float *)p.pl,
                           (const float *)tq->signs, out, nh, splits));
    return IM_OK;
}
}  // namespace im

IM_EXPORT size_t im_cuda_tq_prefill_scratch_bytes(int nkv, int max_seq) { return im::tq_prefill_scratch_bytes(nkv, max_seq); }

// Prefill form of im_cuda_tq_attention for one sequence (cache slot 0): T tokens at positions base_pos .. base_pos + T - 1,
// whose rows are already in the cache; the cached rows are dequantised once into dq_dev and a causal flash-attention
// pass runs over them on the tensor cores (tq_prefill.cu).  Same arithmetic contract and tolerance as im_cuda_tq_attention.
IM_EXPORT int im_cuda_tq_prefill_attention(im_tq *tq, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev, const float *k_scale_dev,
                                           const float *v_scale_dev, const float *k_rnorm_dev, float attn_scale, void *out_dev, int nh, int nkv,
                                           int max_seq, int base_pos, int T, void *dq_dev, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(tq && q_dev && k_cache_dev && v_cache_dev && k_scale_dev && v_scale_dev && k_rnorm_dev && out_dev && dq_dev, "bad argument");
    IM_REQUIRE(tq->hd == kHd, "the attention kernel is built for head_dim 128 (got %d)", tq->hd);
    IM_REQUIRE(nkv > 0 && nh % nkv == 0, "nh must be a multiple of nkv");
    IM_REQUIRE(T >= 0 && max_seq > 0 && base_pos >= 0, "bad shape");
    if (T == 0) return IM_OK;
    if (base_pos + T > max_seq) return fail(IM_ERR_BOUNDS, "sequence position %d + %d tokens exceeds max_seq_len %d", base_pos, T, max_seq);
    const size_t need = im_cuda_tq_scratch_bytes(1, T, nh, kHd, 1);
    if (need > tq->scratch_bytes) {
        int rc = im_cuda_tq_reserve_scratch(tq, need);
        if (rc != IM_OK) return rc;
    }
    float *qrot = tq->scratch + tq_partial_bytes(1, T, nh, kHd, 1) / sizeof(float);
    IM_CUDA_CHECK(launch_k(tq_qrot_kernel, dim3(T, nh), dim3(kHd), 0, as_stream(stream), static_cast<const __half *>(q_dev), (const float *)tq->signs,
                           (const float *)tq->qjl_t, qrot, nh));
    const int rc = tq_prefill_attention_launch(tq, tq->scratch, dq_dev, qrot, static_cast<const uint8_t *>(k_cache_dev), static_cast<const uint8_t *>(v_cache_dev),
                                               k_scale_dev, v_scale_dev, k_rnorm_dev, attn_scale, static_cast<__half *>(out_dev), 0, nh, nkv, max_seq, nullptr, T,
                                               base_pos + T, as_stream(stream), base_pos);
    if (rc == IM_ERR_BOUNDS) return fail(IM_ERR_INVALID, "query heads per KV head must be 1, 2, 4 or 8 (got %d/%d)", nh, nkv);
    return rc;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_tq_attention(im_tq *tq, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                   const float *k_scale_dev, const float *v_scale_dev, const float *k_rnorm_dev, float attn_scale,
                                   void *out_dev, int nseq, int nh, int nkv, int max_seq, int base_pos, const int *pos_dev, int T,
                                   int num_splits, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(tq && q_dev && k_cache_dev && v_cache_dev && k_scale_dev && v_scale_dev && k_rnorm_dev && out_dev, "bad argument");
    IM_REQUIRE(tq->hd == kHd, "the attention kernel is built for head_dim 128 (got %d)", tq->hd);
    IM_REQUIRE(nkv > 0 && nh % nkv == 0, "nh must be a multiple of nkv");
    IM_REQUIRE(nseq >= 0 && T >= 0 && max_seq > 0 && base_pos >= 0, "bad shape");
    if (nseq == 0 || T == 0) return IM_OK;
    if (!pos_dev && base_pos + T > max_seq)
        return fail(IM_ERR_BOUNDS, "sequence position %d + %d tokens exceeds max_seq_len %d", base_pos, T, max_seq);
    int splits = num_splits > 0 ? num_splits : tq_auto_splits(tq->dev, nseq, T, nkv, base_pos + T);
    IM_REQUIRE(splits <= 1024, "too many splits");
    const size_t need = im_cuda_tq_scratch_bytes(nseq, T, nh, kHd, splits);
    if (need > tq->scratch_bytes) {
        int rc = im_cuda_tq_reserve_scratch(tq, need);
        if (rc != IM_OK) return rc;
    }
    // rotate the queries once (every split of a head would otherwise redo the rotation and the 128 x 128 projection)
    float *qrot = tq->scratch + tq_partial_bytes(nseq, T, nh, kHd, splits) / sizeof(float);
    IM_CUDA_CHECK(launch_k(tq_qrot_kernel, dim3(nseq * T, nh), dim3(kHd), 0, as_stream(stream), static_cast<const __half *>(q_dev),
                           (const float *)tq->signs, (const float *)tq->qjl_t, qrot, nh));
    return tq_attention_launch(tq, tq->scratch, nullptr, static_cast<const uint8_t *>(k_cache_dev),
                               static_cast<const uint8_t *>(v_cache_dev), k_scale_dev, v_scale_dev, k_rnorm_dev, attn_scale,
                               static_cast<__half *>(out_dev), nseq, nh, nkv, max_seq, base_pos, pos_dev, T, splits, as_stream(stream), qrot);
    IM_GUARD_END
}

// Fused form of (fused_qk_norm_rope | rope) + turboquant_cache_write(K) + turboquant_cache_write(V) + the query
// rotation of turboquant_attention, followed by the attention itself; one call for the engine and the tests.
IM_EXPORT int im_cuda_tq_fused_attention(im_tq *tq, const void *qkv_dev, int qkv_stride, int k_offset, int v_offset,
                                         const void *q_norm_w_dev, const void *k_norm_w_dev, const void *cos_dev, const void *sin_dev,
                                         int rotary_dim, float eps, void *k_cache_dev, void *v_cache_dev, float *k_scale_dev,
                                         float *v_scale_dev, float *k_rnorm_dev, float attn_scale, float *qrot_dev, void *out_dev,
                                         int nseq, int nh, int nkv, int max_seq, int base_pos, const int *pos_dev, int T,
                                         int num_splits, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(tq && qkv_dev && cos_dev && sin_dev && k_cache_dev && v_cache_dev && k_scale_dev && v_scale_dev && k_rnorm_dev &&
                   qrot_dev && out_dev, "bad argument");
    IM_REQUIRE(tq->hd == kHd, "built for head_dim 128 (got %d)", tq->hd);
    IM_REQUIRE(nkv > 0 && nh % nkv == 0, "nh must be a multiple of nkv");
    IM_REQUIRE((q_norm_w_dev == nullptr) == (k_norm_w_dev == nullptr), "give both norm weights or neither");
    if (nseq == 0 || T == 0) return IM_OK;
    if (!pos_dev && base_pos + T > max_seq)
        return fail(IM_ERR_BOUNDS, "sequence position %d + %d tokens exceeds max_seq_len %d", base_pos, T, max_seq);
    const int splits = num_splits > 0 ? num_splits : tq_auto_splits(tq->dev, nseq, T, nkv, base_pos + T);
    const size_t need = im_cuda_tq_scratch_bytes(nseq, T, nh, kHd, splits);
    if (need > tq->scratch_bytes) {
        int rc = im_cuda_tq_reserve_scratch(tq, need);
        if (rc != IM_OK) return rc;
    }
    TqPrep a{};
    a.qkv = static_cast<const __half *>(qkv_dev); a.stride = qkv_stride; a.k_off = k_offset; a.v_off = v_offset;
    a.qw = static_cast<const __half *>(q_norm_w_dev); a.kw = static_cast<const __half *>(k_norm_w_dev);
    a.cosc = static_cast<const __half *>(cos_dev); a.sinc = static_cast<const __half *>(sin_dev);
    a.nh = nh; a.nkv = nkv; a.rotary_dim = rotary_dim; a.with_norm = q_norm_w_dev != nullptr; a.T = T; a.nseq = nseq;
    a.max_seq = max_seq; a.base_pos = base_pos; a.eps = eps; a.pos_dev = pos_dev; a.qrot = qrot_dev;
    a.kc = static_cast<uint8_t *>(k_cache_dev); a.vc = static_cast<uint8_t *>(v_cache_dev);
    a.ks = k_scale_dev; a.vs = v_scale_dev; a.krn = k_rnorm_dev;
    cudaStream_t st = as_stream(stream);
    int rc = tq_prep_launch(tq, a, st);
    if (rc != IM_OK) return rc;
    return tq_attention_launch(tq, tq->scratch, nullptr, a.kc, a.vc, a.ks, a.vs, a.krn, attn_scale, static_cast<__half *>(out_dev), nseq,
                               nh, nkv, max_seq, base_pos, pos_dev, T, splits, st, qrot_dev);
    IM_GUARD_END
}

// ---------------------------------------------------------------- attention without any allocation
// Some hosts cannot allocate device memory at the moment they need attention: a serving loop that has handed
// all memory to its own arena, code running between the capture and the replay of someone else's CUDA graph, a
// plugin whose host forbids cudaMalloc after start-up.  For them the split partials live in a fixed array that
// is part of the library image: every GPU that loads the library holds these 4 MiB until the process exits.
constexpr size_t kStaticScratchFloats = (size_t)1 << 20;  // 4 MiB
static __device__ __align__(256) float g_static_attn_scratch[kStaticScratchFloats];
static float *g_static_attn_ptr[64] = {};  // device address of the array, per device ordinal

IM_EXPORT int im_cuda_tq_attention_static(const im_tq *tq, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                          const float *k_scale_dev, const float *v_scale_dev, const float *k_rnorm_dev,
                                          float attn_scale, void *out_dev, int nseq, int nh, int nkv, int max_seq, int base_pos,
                                          const int *pos_dev, int T, int num_splits, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(tq && q_dev && k_cache_dev && v_cache_dev && k_scale_dev && v_scale_dev && k_rnorm_dev && out_dev, "bad argument");
    IM_REQUIRE(tq->hd == kHd, "the attention kernel is built for head_dim 128 (got %d)", tq->hd);
    IM_REQUIRE(nkv > 0 && nh % nkv == 0, "nh must be a multiple of nkv");
    IM_REQUIRE(nseq >= 0 && T >= 0 && max_seq > 0 && base_pos >= 0, "bad shape");
    if (nseq == 0 || T == 0) return IM_OK;
    if (!pos_dev && base_pos + T > max_seq)
        return fail(IM_ERR_BOUNDS, "sequence position %d + %d tokens exceeds max_seq_len %d", base_pos, T, max_seq);
    int cur = -1;
    IM_CUDA_CHECK(cudaGetDevice(&cur));
    IM_REQUIRE(cur == tq->dev->ordinal, "device %d must be current (device %d is)", tq->dev->ordinal, cur);
    IM_REQUIRE(cur >= 0 && cur < 64, "device ordinal %d is outside the table", cur);
    if (!g_static_attn_ptr[cur]) {
        // The array's name is a host-side stand-in; the kernels need its address on THIS device.
        float *ptr = nullptr;
        IM_CUDA_CHECK(cudaGetSymbolAddress((void **)&ptr, g_static_attn_scratch));
        g_static_attn_ptr[cur] = ptr;
    }
    // The array holds what im_cuda_tq_attention keeps in its allocated scratch: the split partials, then the rotated
    // queries of the pre-pass (so both entry points run the same kernels).  A split count chosen here shrinks until
    // the request fits; one given by the caller is taken as it is or refused.
    int splits = num_splits > 0 ? num_splits : tq_auto_splits(tq->dev, nseq, T, nkv, base_pos + T);
    while (num_splits <= 0 && splits > 1 && im_cuda_tq_scratch_bytes(nseq, T, nh, kHd, splits) > kStaticScratchFloats * sizeof(float)) splits--;
    const size_t need = im_cuda_tq_scratch_bytes(nseq, T, nh, kHd, splits);
    if (need > kStaticScratchFloats * sizeof(float))
        return fail(IM_ERR_BOUNDS,
                    "%d sequence(s) x %d token(s) x %d heads x %d splits need %zu bytes of split partials and rotated queries; the built-in "
                    "scratch holds %zu (use fewer splits or im_cuda_tq_attention)",
                    nseq, T, nh, splits, need, kStaticScratchFloats * sizeof(float));
    // Nothing has to start at zero: every split, empty ones included, writes its whole partial before the reduce reads it.
    float *scratch = g_static_attn_ptr[cur];
    float *qrot = scratch + tq_partial_bytes(nseq, T, nh, kHd, splits) / sizeof(float);
    IM_CUDA_CHECK(launch_k(tq_qrot_kernel, dim3(nseq * T, nh), dim3(kHd), 0, as_stream(stream), static_cast<const __half *>(q_dev),
                           (const float *)tq->signs, (const float *)tq->qjl_t, qrot, nh));
    return tq_attention_launch(tq, scratch, nullptr, static_cast<const uint8_t *>(k_cache_dev),
                               static_cast<const uint8_t *>(v_cache_dev), k_scale_dev, v_scale_dev, k_rnorm_dev, attn_scale,
                               static_cast<__half *>(out_dev), nseq, nh, nkv, max_seq, base_pos, pos_dev, T, splits, as_stream(stream), qrot);
    IM_GUARD_END
}
