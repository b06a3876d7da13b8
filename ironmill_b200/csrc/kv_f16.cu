// Attention over an unquantized fp16 KV cache: the reference's path with TurboQuant switched off
// (crates/ironmill-inference/src/metal/attention.rs:491-612):
//   kv_scatter             shaders/kv/kv_scatter.metal:20-42            K / V projections -> cache [nkv, max_seq, hd]
//   fused_sdpa             shaders/attention/fused_sdpa.metal:52-251    decode, short contexts
//   prefill_attention_v2   shaders/attention/attention.metal:571-750    more than one token (causal)
//   fused_sdpa_split + fused_sdpa_reduce   shaders/attention/flash_decode.metal:25-215   decode, long contexts
// All of them compute softmax(scale * q . K^T) V with fp16 inputs, f32 scores / online softmax / accumulation and one
// fp16 rounding of the output; they differ in tiling only.  Here one kernel covers them: a warp per query head walks
// its share of the cached positions in tiles of 32 (lane = position for the scores, lane = four dimensions for the
// weighted sum), the query heads of a KV head share a CTA (their K / V tiles are staged once in shared memory), grid z
// splits the positions of long contexts and a reduction kernel combines the splits exactly as fused_sdpa_reduce does.
// Prefill chunks of one sequence (16 tokens and more) take a causal tensor-core pass instead (sdpa16_prefill_kernel).
#include <algorithm>

#include "common.cuh"

namespace im {

namespace {

constexpr int kHd16 = 128;
constexpr int kTile16 = 32;

__device__ __forceinline__ int slot_of(const int *slot_map, int seq) { return slot_map ? slot_map[seq] : seq; }

// (QK-norm,) RoPE, cache write.  One CTA of 128 threads per (token, head): query heads are rounded to fp16 in place
// (the reference's q_proj buffer after fused_qk_norm_rope / rope), key heads are rounded and scattered, value heads are
// scattered as they are.
__global__ void __launch_bounds__(kHd16) kv16_prep_kernel(const Kv16Prep a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sh[kHd16];
    __shared__ float red[4];
    const int st = blockIdx.x, slot = blockIdx.y, d = threadIdx.x;
    const int seq = slot_of(a.slot_map, st / a.T), t = st % a.T;
    const int pos_abs = a.base_pos + (a.pos_dev ? a.pos_dev[seq] : 0) + t;
    __half *tok = a.qkv + (size_t)st * a.stride;
    const __half *tokkv = a.kv ? a.kv + (size_t)st * a.kv_stride : tok;
    if (slot >= a.nh + a.nkv) {  // value head
        const int h = slot - a.nh - a.nkv;
        const size_t row = ((size_t)seq * a.nkv + h) * a.max_seq + pos_abs % a.max_seq;
        a.vc[row * kHd16 + d] = tokkv[a.v_off + h * kHd16 + d];
        return;
    }
    const bool is_q = slot < a.nh;
    const int h = is_q ? slot : slot - a.nh;
    const __half *src = (is_q ? tok : tokkv + a.k_off) + h * kHd16;
    const __half *w = is_q ? a.qw : a.kw;
    float x = __half2float(src[d]);
    const int half_rot = a.rotary_dim / 2;
    const int ri = d < half_rot ? d : d - half_rot;
    float rc = 1.0f, rs = 0.0f;
    if (d < a.rotary_dim) {
        rc = __half2float(a.cosc[(size_t)pos_abs * (kHd16 / 2) + ri]);
        rs = __half2float(a.sinc[(size_t)pos_abs * (kHd16 / 2) + ri]);
    }
    if (a.with_norm) {
        const float ss = warp_sum(x * x);
        if ((d & 31) == 0) red[d >> 5] = ss;
        __syncthreads();
        const float tot = red[0] + red[1] + red[2] + red[3];
        x = x * rsqrtf(tot / (float)kHd16 + a.eps) * __half2float(w[d]);
    }
    sh[d] = x;
    __syncthreads();
    float y = x;
    if (d < a.rotary_dim) {
        const float lo = sh[ri], hi = sh[ri + half_rot];
        y = d < half_rot ? lo * rc - hi * rs : lo * rs + hi * rc;
    }
    const __half yh = __float2half_rn(y);
    if (is_q) {
        tok[h * kHd16 + d] = yh;
    } else {
        const size_t row = ((size_t)seq * a.nkv + h) * a.max_seq + pos_abs % a.max_seq;
        a.kc[row * kHd16 + d] = yh;
    }
}

// kv_scatter alone (the reference's kernel): proj [nseq*T, nkv, hd] -> cache rows at the tokens' positions.
__global__ void kv16_scatter_kernel(const __half *__restrict__ proj, __half *__restrict__ cache, int T, int nkv, int max_seq, int base_pos,
                                    const int *__restrict__ pos_dev, const int *__restrict__ slot_map) {
    const int st = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const int seq = slot_of(slot_map, st / T), t = st % T;
    const int pos = (base_pos + (pos_dev ? pos_dev[seq] : 0) + t) % max_seq;
    cache[(((size_t)seq * nkv + h) * max_seq + pos) * kHd16 + d] = proj[((size_t)st * nkv + h) * kHd16 + d];
}

struct Sdpa16 {
    const __half *q;   // query of (token st, head h) at q + st * q_stride + h * hd
    int q_stride;
    const __half *kc, *vc;  // [slots, nkv, max_seq, hd]
    __half *out;       // [nseq*T, nh, hd]
    float *po, *pm, *pl;  // split partials [nseq*T*nh, splits] (x hd for po)
    int nh, nkv, T, max_seq, base_pos, splits;
    const int *pos_dev, *slot_map;
    float scale;
};

// grid (nseq*T, nkv, splits), block GQ warps: warp w = query head kvh * GQ + w.  The CTA brings each tile of 32 K rows
// and 32 V rows into shared memory once (16-byte asynchronous copies, two tiles in flight) for all of its query heads;
// K rows sit 272 bytes apart so that a lane reading its own row with 128-bit loads meets no bank conflict.
constexpr int kKRow16 = 272, kVRow16 = 256;

template <int GQ>
__global__ void __launch_bounds__(GQ * 32) sdpa16_kernel(const Sdpa16 p) {
    pdl_trigger();
    pdl_wait();
    constexpr int NT = GQ * 32;
    __shared__ __align__(16) unsigned char ksm[2][kTile16 * kKRow16];
    __shared__ __align__(16) unsigned char vsm[2][kTile16 * kVRow16];
    __shared__ __align__(16) float qs[GQ][kHd16];
    const int st = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = kvh * GQ + warp;
    const int seq = slot_of(p.slot_map, st / p.T), t = st % p.T;
    // positions this token attends to: everything cached before it and itself (causal), never past the cache
    const int seq_len = min(p.base_pos + (p.pos_dev ? p.pos_dev[seq] : 0) + t + 1, p.max_seq);
    int chunk = (seq_len + p.splits - 1) / p.splits;
    chunk = (chunk + kTile16 - 1) / kTile16 * kTile16;
    const int r0 = split * chunk, r1 = min(r0 + chunk, seq_len);
    {
        const __half *qp = p.q + (size_t)st * p.q_stride + (size_t)head * kHd16;
        const uint2 raw = *reinterpret_cast<const uint2 *>(qp + 4 * lane);
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
        *reinterpret_cast<float4 *>(&qs[warp][4 * lane]) = make_float4(a.x, a.y, b.x, b.y);
    }
    const size_t cache_base = ((size_t)seq * p.nkv + kvh) * p.max_seq * kHd16;
    auto load_tile = [&](int buf, int tile) {  // rows past the split's end repeat its last row (their weights are zero)
        for (int c = threadIdx.x; c < kTile16 * 16; c += NT) {
            const int row = c >> 4, ch = c & 15;
            const size_t src = cache_base + (size_t)min(tile + row, r1 - 1) * kHd16 + ch * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(&ksm[buf][row * kKRow16 + ch * 16])), "l"(p.kc + src) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(&vsm[buf][row * kVRow16 + ch * 16])), "l"(p.vc + src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float m = -INFINITY, l = 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const int ntiles = r1 > r0 ? (r1 - r0 + kTile16 - 1) / kTile16 : 0;
    if (ntiles > 0) load_tile(0, r0);
    for (int it = 0; it < ntiles; it++) {
        const int tile = r0 + it * kTile16, buf = it & 1;
        if (it + 1 < ntiles) {
            load_tile(buf ^ 1, tile + kTile16);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // the tile (and, the first time, the queries) is visible to every warp
        const bool live = tile + lane < r1;
        float s = -INFINITY;
        {
            const uint4 *kr = reinterpret_cast<const uint4 *>(&ksm[buf][lane * kKRow16]);
            float dot = 0.0f;
#pragma unroll 4
            for (int i = 0; i < kHd16 / 8; i++) {
                const uint4 raw = kr[i];
                const float4 q0 = *reinterpret_cast<const float4 *>(&qs[warp][8 * i]), q1 = *reinterpret_cast<const float4 *>(&qs[warp][8 * i + 4]);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x)), k1 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.z)), k3 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.w));
                dot = fmaf(q0.x, k0.x, dot); dot = fmaf(q0.y, k0.y, dot); dot = fmaf(q0.z, k1.x, dot); dot = fmaf(q0.w, k1.y, dot);
                dot = fmaf(q1.x, k2.x, dot); dot = fmaf(q1.y, k2.y, dot); dot = fmaf(q1.z, k3.x, dot); dot = fmaf(q1.w, k3.y, dot);
            }
            if (live) s = dot * p.scale;
        }
        float tmax = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        if (tmax > m) {  // the reference rescales only when the maximum moves
            const float corr = __expf(m - tmax);  // exp(-inf) = 0 on the first tile
            l *= corr;
#pragma unroll
            for (int j = 0; j < 4; j++) acc[j] *= corr;
            m = tmax;
        }
        const float wgt = live ? __expf(s - m) : 0.0f;
        l += warp_sum(wgt);
        const unsigned char *vr = &vsm[buf][8 * lane];
#pragma unroll 8
        for (int j = 0; j < kTile16; j++) {  // rows past the end carry weight zero
            const float wj = __shfl_sync(0xffffffffu, wgt, j);
            const uint2 raw = *reinterpret_cast<const uint2 *>(vr + j * kVRow16);
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
            acc[0] = fmaf(wj, a.x, acc[0]); acc[1] = fmaf(wj, a.y, acc[1]); acc[2] = fmaf(wj, b.x, acc[2]); acc[3] = fmaf(wj, b.y, acc[3]);
        }
        __syncthreads();  // every warp is done with this buffer before the copies of the tile after next land in it
    }
    const size_t hidx = (size_t)st * p.nh + head;
    if (p.splits == 1) {
        const float inv = 1.0f / fmaxf(l, 1e-10f);
        const __half2 lo = __floats2half2_rn(acc[0] * inv, acc[1] * inv), hi = __floats2half2_rn(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2 *>(p.out + hidx * kHd16 + 4 * lane) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    } else {  // unnormalised partial of this split (an empty split leaves max = -inf, sum = 0)
        const size_t pi = hidx * p.splits + split;
        *reinterpret_cast<float4 *>(p.po + pi * kHd16 + 4 * lane) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (lane == 0) {
            p.pm[pi] = m;
            p.pl[pi] = l;
        }
    }
}

// ---- prefill chunks of one sequence (prefill_attention_v2, attention.metal:571-750): causal flash attention on the
// tensor cores.  A CTA owns 16 consecutive tokens of one KV head = 16 * GQ score rows (row = token * GQ + head), one warp
// per 16 rows (mma.sync m16n8k16, operands by ldmatrix); K / V tiles of 32 cached rows by 16-byte cp.async into
// shared-memory rows 272 bytes apart, two tiles in flight.  fp16 operands (the cache and the queries are fp16 already; the
// softmax weights are rounded to fp16 for the second product), f32 scores, sums and outputs.
constexpr int kPf16Tok = 16, kPf16N = 32, kPf16Row = 272;
__device__ __forceinline__ void mma16816_f(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ unsigned pack_h2f(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&h);
}

// grid (ceil(T / 16), nkv); block GQ warps; one sequence (cache slot `slot`), T tokens at positions P .. P + T - 1.
template <int GQ>
__global__ void __launch_bounds__(GQ * 32, GQ == 8 ? 1 : 2) sdpa16_prefill_kernel(const Sdpa16 p, int slot) {
    constexpr int M = kPf16Tok * GQ, NT = GQ * 32;
    extern __shared__ __align__(16) unsigned char pf16_smem[];
    unsigned char *qs = pf16_smem;                      // [M][272]
    unsigned char *kt = qs + M * kPf16Row;              // [2][32][272]
    unsigned char *vt = kt + 2 * kPf16N * kPf16Row;     // [2][32][272]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int tb = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y;  // longest (latest) token blocks first
    pdl_trigger();
    pdl_wait();
    const int P = p.base_pos + (p.pos_dev ? p.pos_dev[slot] : 0);
    for (int i = tid; i < M * 16; i += NT) {
        const int r = i >> 4, c = i & 15;
        const int tok = tb * kPf16Tok + r / GQ, h = kvh * GQ + r % GQ;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < p.T) v = *reinterpret_cast<const uint4 *>(p.q + (size_t)tok * p.q_stride + (size_t)h * kHd16 + 8 * c);
        *reinterpret_cast<uint4 *>(qs + r * kPf16Row + 16 * c) = v;
    }
    const int last_tok = min(tb * kPf16Tok + kPf16Tok - 1, p.T - 1);
    const int n_end = min(P + last_tok + 1, p.max_seq);
    const int ntiles = (n_end + kPf16N - 1) / kPf16N;
    const size_t cache_base = ((size_t)slot * p.nkv + kvh) * p.max_seq * kHd16;
    auto load_tile = [&](int buf, int tile) {
        const int p0 = tile * kPf16N;
        for (int i = tid; i < kPf16N * 16; i += NT) {
            const int r = i >> 4, c = i & 15;
            const size_t src = cache_base + (size_t)min(p0 + r, n_end - 1) * kHd16 + 8 * c;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(kt + (buf * kPf16N + r) * kPf16Row + 16 * c)), "l"(p.kc + src) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(vt + (buf * kPf16N + r) * kPf16Row + 16 * c)), "l"(p.vc + src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int row0 = warp * 16 + g, row1 = row0 + 8;
    const int tok0 = tb * kPf16Tok + row0 / GQ, tok1 = tb * kPf16Tok + row1 / GQ;
    const int lim0 = tok0 < p.T ? P + tok0 : -1, lim1 = tok1 < p.T ? P + tok1 : -1;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const unsigned qs_a = (unsigned)__cvta_generic_to_shared(qs + (warp * 16 + (lane & 15)) * kPf16Row + (lane >> 4) * 16);
    if (ntiles > 0) load_tile(0, 0);
    for (int it = 0; it < ntiles; it++) {
        const int buf = it & 1, p0 = it * kPf16N;
        if (it + 1 < ntiles) {
            load_tile(buf ^ 1, it + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        float sc[4][4];
#pragma unroll
        for (int nb = 0; nb < 4; nb++) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.0f;
        const unsigned kt_a = (unsigned)__cvta_generic_to_shared(kt + (buf * kPf16N + (lane & 7) + 8 * (lane >> 4)) * kPf16Row + ((lane >> 3) & 1) * 16);
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
            unsigned a[4], b01[4], b23[4];
            ldsm4(a, qs_a + kk * 32);
            ldsm4(b01, kt_a + kk * 32);
            ldsm4(b23, kt_a + 16 * kPf16Row + kk * 32);
            mma16816_f(sc[0], a[0], a[1], a[2], a[3], b01[0], b01[1]);
            mma16816_f(sc[1], a[0], a[1], a[2], a[3], b01[2], b01[3]);
            mma16816_f(sc[2], a[0], a[1], a[2], a[3], b23[0], b23[1]);
            mma16816_f(sc[3], a[0], a[1], a[2], a[3], b23[2], b23[3]);
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 4; nb++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int pos = p0 + 8 * nb + 2 * t + (e & 1);
                const int lim = (e < 2) ? lim0 : lim1;
                sc[nb][e] = (pos <= lim && pos < n_end) ? sc[nb][e] * p.scale : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], sc[nb][e]);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = m_new == -INFINITY ? 1.0f : __expf(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        unsigned pa[2][4];
#pragma unroll
        for (int nb = 0; nb < 4; nb++) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                w[e] = sc[nb][e] == -INFINITY ? 0.0f : __expf(sc[nb][e] - m_run[e >> 1]);
                l_run[e >> 1] += w[e];
            }
            pa[nb >> 1][(nb & 1) * 2 + 0] = pack_h2f(w[0], w[1]);
            pa[nb >> 1][(nb & 1) * 2 + 1] = pack_h2f(w[2], w[3]);
        }
#pragma unroll
        for (int kb = 0; kb < 2; kb++) {
            const unsigned vt_a = (unsigned)__cvta_generic_to_shared(vt + (buf * kPf16N + 16 * kb + (lane & 15)) * kPf16Row + (lane >> 4) * 16);
#pragma unroll
            for (int nd = 0; nd < 16; nd += 2) {
                unsigned b[4];
                ldsm4_t(b, vt_a + nd * 16);
                mma16816_f(o[nd], pa[kb][0], pa[kb][1], pa[kb][2], pa[kb][3], b[0], b[1]);
                mma16816_f(o[nd + 1], pa[kb][0], pa[kb][1], pa[kb][2], pa[kb][3], b[2], b[3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        const int row = r == 0 ? row0 : row1, tok = r == 0 ? tok0 : tok1;
        if (tok < p.T) {
            const float inv = 1.0f / fmaxf(l_run[r], 1e-10f);
            __half *dst = p.out + ((size_t)tok * p.nh + kvh * GQ + row % GQ) * kHd16;
#pragma unroll
            for (int nd = 0; nd < 16; nd++) *reinterpret_cast<unsigned *>(dst + 8 * nd + 2 * t) = pack_h2f(o[nd][2 * r] * inv, o[nd][2 * r + 1] * inv);
        }
    }
}

template <int GQ>
static int sdpa16_prefill_launch(const Sdpa16 &p, int slot, const Device *dev, cudaStream_t st) {
    constexpr size_t smem = (size_t)kPf16Tok * GQ * kPf16Row + 4 * kPf16N * kPf16Row;
    auto kern = sdpa16_prefill_kernel<GQ>;
    static DeviceOnce once;
    if (once.first(dev->ordinal)) IM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    IM_CUDA_CHECK(launch_k(kern, dim3((p.T + kPf16Tok - 1) / kPf16Tok, p.nkv), dim3(GQ * 32), smem, st, p, slot));
    return IM_OK;
}

// fused_sdpa_reduce (flash_decode.metal:163-215): global max over the splits, rescale, normalise, fp16.
__global__ void __launch_bounds__(kHd16) sdpa16_reduce_kernel(const float *__restrict__ po, const float *__restrict__ pm, const float *__restrict__ pl,
                                                              __half *__restrict__ out, int splits) {
    pdl_trigger();
    pdl_wait();
    const size_t hidx = blockIdx.x;
    const int d = threadIdx.x;
    float gm = -INFINITY;
    for (int s = 0; s < splits; s++) gm = fmaxf(gm, pm[hidx * splits + s]);
    float acc = 0.0f, lsum = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float mv = pm[hidx * splits + s];
        const float corr = mv == -INFINITY ? 0.0f : __expf(mv - gm);
        lsum += pl[hidx * splits + s] * corr;
        acc += po[(hidx * splits + s) * kHd16 + d] * corr;
    }
    out[hidx * kHd16 + d] = __float2half_rn(acc / fmaxf(lsum, 1e-10f));
}

}  // namespace

size_t kv16_scratch_bytes(int tokens, int nh, int splits) { return (size_t)tokens * nh * splits * (kHd16 + 2) * sizeof(float); }

// Splits for a launch: one when the (token, KV head) pairs already fill the GPU or the context is short (the reference's
// single-pass kernels), otherwise enough to give every SM two CTAs, at least 256 positions each.
int kv16_auto_splits(const Device *dev, int tokens, int nkv, int max_ctx) {
    const int ctas = tokens * nkv;
    if (ctas >= dev->sm_count || max_ctx < 256) return 1;
    int s = (2 * dev->sm_count + ctas - 1) / ctas;
    s = std::min(s, (max_ctx + 255) / 256);
    return std::max(1, std::min(s, 64));
}

int kv16_prep_launch(const Kv16Prep &a, cudaStream_t st) {
    if (a.nseq * a.T == 0) return IM_OK;
    IM_CUDA_CHECK(launch_k(kv16_prep_kernel, dim3(a.nseq * a.T, a.nh + 2 * a.nkv), dim3(kHd16), 0, st, a));
    return IM_OK;
}

int kv16_attention_launch(const Device *dev, float *scratch, size_t scratch_bytes, const __half *q, int q_stride, const __half *kc, const __half *vc,
                          float scale, __half *out, int nseq, int nh, int nkv, int max_seq, int base_pos, const int *pos_dev, int T, int splits,
                          int ctx_hint, cudaStream_t st, const int *slot_map, int prefill_slot) {
    const int tokens = nseq * T;
    if (tokens == 0) return IM_OK;
    if (nkv <= 0 || nh % nkv != 0) return fail(IM_ERR_INVALID, "nh must be a multiple of nkv");
    const int gq = nh / nkv;
    if (gq != 1 && gq != 2 && gq != 4 && gq != 8) return fail(IM_ERR_INVALID, "fp16-KV attention is built for 1, 2, 4 or 8 query heads per KV head (got %d)", gq);
    if (nseq == 1 && T >= 16 && prefill_slot >= 0) {  // a prefill chunk of one sequence (cache slot known to the host): the tensor-core pass
        Sdpa16 f{};
        f.q = q; f.q_stride = q_stride; f.kc = kc; f.vc = vc; f.out = out; f.nh = nh; f.nkv = nkv; f.T = T; f.max_seq = max_seq;
        f.base_pos = base_pos; f.pos_dev = pos_dev; f.scale = scale; f.splits = 1;
        switch (gq) {
        case 1: return sdpa16_prefill_launch<1>(f, prefill_slot, dev, st);
        case 2: return sdpa16_prefill_launch<2>(f, prefill_slot, dev, st);
        case 4: return sdpa16_prefill_launch<4>(f, prefill_slot, dev, st);
        default: return sdpa16_prefill_launch<8>(f, prefill_slot, dev, st);
        }
    }
    if (splits <= 0) splits = kv16_auto_splits(dev, tokens, nkv, ctx_hint > 0 ? ctx_hint : max_seq);
    while (splits > 1 && kv16_scratch_bytes(tokens, nh, splits) > scratch_bytes) splits--;
    Sdpa16 p{};
    p.q = q; p.q_stride = q_stride; p.kc = kc; p.vc = vc; p.out = out;
    p.po = scratch;
    p.pm = scratch + (size_t)tokens * nh * splits * kHd16;
    p.pl = p.pm + (size_t)tokens * nh * splits;
    p.nh = nh; p.nkv = nkv; p.T = T; p.max_seq = max_seq; p.base_pos = base_pos; p.splits = splits;
    p.pos_dev = pos_dev; p.slot_map = slot_map; p.scale = scale;
    const dim3 grid(tokens, nkv, splits);
    switch (gq) {
    case 1: IM_CUDA_CHECK(launch_k(sdpa16_kernel<1>, grid, dim3(32), 0, st, p)); break;
    case 2: IM_CUDA_CHECK(launch_k(sdpa16_kernel<2>, grid, dim3(64), 0, st, p)); break;
    case 4: IM_CUDA_CHECK(launch_k(sdpa16_kernel<4>, grid, dim3(128), 0, st, p)); break;
    default: IM_CUDA_CHECK(launch_k(sdpa16_kernel<8>, grid, dim3(256), 0, st, p)); break;
    }
    if (splits > 1)
        IM_CUDA_CHECK(launch_k(sdpa16_reduce_kernel, dim3((unsigned)((size_t)tokens * nh)), dim3(kHd16), 0, st, (const float *)p.po, (const float *)p.pm,
                               (const float *)p.pl, out, splits));
    return IM_OK;
}

}  // namespace im

// ---- C ABI ------------------------------------------------------------------------------------------------------
IM_EXPORT int im_cuda_kv_scatter_f16(const void *proj_dev, void *cache_dev, int nseq, int T, int nkv, int head_dim, int max_seq, int base_pos,
                                     const int *pos_dev, const int *slot_map_dev, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(proj_dev && cache_dev, "bad argument");
    IM_REQUIRE(head_dim == im::kHd16, "the fp16-KV kernels are built for head_dim 128 (got %d)", head_dim);
    IM_REQUIRE(nseq >= 0 && T >= 0 && nkv > 0 && max_seq > 0 && base_pos >= 0, "bad shape");
    if (nseq * T == 0) return IM_OK;
    im::kv16_scatter_kernel<<<dim3(nseq * T, nkv), im::kHd16, 0, im::as_stream(stream)>>>(static_cast<const __half *>(proj_dev), static_cast<__half *>(cache_dev), T,
                                                                                       nkv, max_seq, base_pos, pos_dev, slot_map_dev);
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT size_t im_cuda_sdpa_f16_scratch_bytes(int nseq, int T, int nh, int splits) { return im::kv16_scratch_bytes(nseq * T, nh, splits < 1 ? 1 : splits); }

IM_EXPORT int im_cuda_sdpa_f16(im_device *dev, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev, void *out_dev, int nseq, int nh,
                               int nkv, int head_dim, int max_seq, int base_pos, const int *pos_dev, int T, float scale, int num_splits,
                               void *scratch_dev, size_t scratch_bytes, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(dev && q_dev && k_cache_dev && v_cache_dev && out_dev, "bad argument");
    IM_REQUIRE(head_dim == im::kHd16, "the fp16-KV kernels are built for head_dim 128 (got %d)", head_dim);
    IM_REQUIRE(nseq >= 0 && T >= 0 && max_seq > 0 && base_pos >= 0, "bad shape");
    IM_REQUIRE(num_splits <= 1 || scratch_dev, "split attention needs a scratch buffer (im_cuda_sdpa_f16_scratch_bytes)");
    if (!scratch_dev) num_splits = 1;
    return im::kv16_attention_launch(dev, static_cast<float *>(scratch_dev), scratch_bytes, static_cast<const __half *>(q_dev), nh * head_dim,
                                     static_cast<const __half *>(k_cache_dev), static_cast<const __half *>(v_cache_dev), scale,
                                     static_cast<__half *>(out_dev), nseq, nh, nkv, max_seq, base_pos, pos_dev, T, num_splits,
                                     pos_dev ? max_seq : base_pos + T,  // positions on the device: the cache length bounds the context
                                     im::as_stream(stream), nullptr, nseq == 1 ? 0 : -1);
    IM_GUARD_END
}
