// Whole-token decode kernel: every decoder layer of one batch-1 decode step in ONE persistent launch.
//
// Why: a decode step of a Llama-3-8B-shaped model is ~230 short kernels (7 per layer).  Each of them pays a
// launch ramp, a pipeline fill and a tail in which HBM idles, and together those fixed costs are several
// times the time the weight bytes need.  Here one CTA per SM lives for the whole token:
//   * its producer warp streams this CTA's share of EVERY projection of EVERY layer, in execution order,
//     through one shared-memory ring with cp.async.bulk.  Weights are constants, so the producer never waits
//     for activations, only for a free ring slot: while the consumers sit in a grid barrier, rotate a query
//     or walk the KV cache, the next projection's tiles are already arriving;
//   * its 16 consumer warps run the phases of the layer (the same arithmetic as the stand-alone kernels:
//     matvec_v2.cu for the projections, tq_device.cuh for RoPE + cache write, attention and its reduction),
//     separated by grid-wide barriers (one arrival counter per barrier, bounded polls).
// Phases of layer l:  [residual+norm ->] QKV | RoPE + TurboQuant cache write + query rotation | split attention
//                     | split reduction | o | residual+norm -> gate/up+SiLU | down.
// The launch is cooperative (all CTAs resident).  Semantics per phase:
//   crates/ironmill-inference/src/metal/pipeline.rs:436-1245 (run_pipeline_inner) and the shader files named in
//   matvec_v2.cu / turboquant.cu.
#include "common.cuh"
#include "tq_device.cuh"
#include "v2_device.cuh"
#include "mega.cuh"

#ifndef IM_MEGA_ITEM_INLINE
#define IM_MEGA_ITEM_INLINE __forceinline__
#endif

namespace im {

namespace {

// x / a for the AWQ scales: approximate reciprocal, product and one Newton step on the remainder, which gives the correctly
// rounded f32 quotient for operands that are not denormal.  (The IEEE division and reciprocal routines cost 6 to 10 us
// per layer of staging time in this kernel: measured.)
__device__ __forceinline__ float div_awq(float x, float a) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));  // one instruction; the Newton step below repairs its last bits
    const float q = x * r;
    return fmaf(fmaf(-q, a, x), r, q);
}

constexpr int kGroups = kV2Consumers / 4;      // 128-thread groups of consumer warps
// 16 consumer warps + the producer warp: five warps share one scheduler's register file, which caps the kernel at 96
// registers per thread.  (Tried: a producer warp GROUP that hands registers to the consumers with setmaxnreg.  The pool
// is what the CTA was launched with, 20 warps x 96, so the consumers reach 112 only if the producer drops to 24-32, and
// a producer that small spills its whole stage walk: 97-101 us per layer against 84 without.)
constexpr int kMegaThreads = kV2Threads;
constexpr int kRedFloats = kV2Consumers * 16;  // per ring slot: 16 row sums from each consumer warp
constexpr int kStageBytes = kStageTiles * kTileBytes;
constexpr int kPhaseWords = sizeof(MegaPhase) / 4, kLayerWords = sizeof(MegaLayer) / 4;
constexpr int kDescWords = (5 * kPhaseWords + kLayerWords + 3) & ~3;  // per layer: phases 4l .. 4l+4, then the layer block

struct Range {
    int t_begin, t_end;
};
__device__ __forceinline__ Range cta_range(int nblk, int G) {  // whole row blocks per CTA
    const int b0 = (int)((long long)nblk * blockIdx.x / gridDim.x), b1 = (int)((long long)nblk * (blockIdx.x + 1) / gridDim.x);
    return Range{b0 * G, b1 * G};
}
// barrier index of matvec phase q (4 per layer: qkv, o, gate/up, down); 7 barriers per layer:
// qkv, prep, attention, reduce, o, gate/up, down
__device__ __forceinline__ int phase_barrier(int q) {
    const int j = q & 3;
    return (q >> 2) * 7 + (j == 0 ? 0 : j + 3);
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_volatile(const int *p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Arrival of this CTA at barrier k: the caller's threads have synchronised among themselves.
__device__ __forceinline__ void grid_arrive(unsigned *bar, int k) {
    // release: the CTA's writes (ordered before this by its own barrier) are visible to whoever acquires the count
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(bar + k), "r"(1u) : "memory");
}
// One thread polls until every CTA has arrived (or the error word is set / the time limit passes).
__device__ __forceinline__ bool grid_poll(const unsigned *bar, int k, int *err, unsigned limit_ms) {
    const unsigned want = gridDim.x;
    if (ld_acquire(bar + k) >= want) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned i = 1;; i++) {  // each poll is a trip to L2: that paces the loop
        if (ld_acquire(bar + k) >= want) return true;
        if ((i & 127u) == 0) {
            if (ld_volatile(err) != 0) return false;
            if (global_ns() - t0 > (unsigned long long)limit_ms * 1000000ull) break;
        }
    }
    atomicExch(err, 2);
    return false;
}

// 16 bytes of a mailbox (two {data, tag} pairs), past every cache
__device__ __forceinline__ uint4 ld_mail(const uint4 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Re-reads one 8-element chunk of a mailbox slot until its four tags match (the writer is another GPU).  Bounded like
// every wait of the kernel: gives up after limit_ms or when the error word is set, and sets it.
__device__ __forceinline__ void mail_settle(const uint4 *src, uint4 &a, uint4 &c, unsigned tag, int *err, unsigned limit_ms) {
    if (a.y == tag && a.w == tag && c.y == tag && c.w == tag) return;
    const unsigned long long t0 = global_ns();
    for (unsigned i = 1;; i++) {
        a = ld_mail(src);
        c = ld_mail(src + 1);
        if (a.y == tag && a.w == tag && c.y == tag && c.w == tag) return;
        if ((i & 127u) == 0) {
            if (ld_volatile(err) != 0) return;
            if (global_ns() - t0 > (unsigned long long)limit_ms * 1000000ull) break;
        }
    }
    atomicExch(err, 2);
}

// ---- activation staging for one batch row (stage_chunk24<1>, v2_device.cuh) ---------------------------------------
__device__ __forceinline__ void unpack2(unsigned w, float &a, float &b) {  // two fp16 values of a word, no address taken
    a = __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
    b = __half2float(__ushort_as_half((unsigned short)(w >> 16)));
}
__device__ __forceinline__ void unpack8(const uint4 raw, float (&v)[8]) {
    unpack2(raw.x, v[0], v[1]);
    unpack2(raw.y, v[2], v[3]);
    unpack2(raw.z, v[4], v[5]);
    unpack2(raw.w, v[6], v[7]);
}

// Plain projection input: x (/ awq).
__device__ __forceinline__ void mega_stage_plain(const __half *__restrict__ x, const __half *__restrict__ awq, int G, uint32_t *xq,
                                                 float2 *meta) {
    const int lane = threadIdx.x & 31, hl = lane & 15, warp = threadIdx.x >> 5;
#pragma unroll 2
    for (int g0 = warp * 2; g0 < G; g0 += kV2Consumers * 2) {
        const int grp = g0 + (lane >> 4);
        const bool live = grp < G;
        const int k = (live ? grp : g0) * 128 + hl * 8;
        const uint4 raw = *reinterpret_cast<const uint4 *>(x + k);
        uint4 ra = make_uint4(0, 0, 0, 0);
        if (awq) ra = *reinterpret_cast<const uint4 *>(awq + k);
        float v[8];
        unpack8(raw, v);
        if (awq) {
            float a[8];
            unpack8(ra, a);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = div_awq(v[i], a[i]);  // f32(x) / f32(awq), as affine_matvec.metal:48-66
        }
        stage_chunk24<1>(v, live, grp, 0, hl, xq, meta);
    }
}

// Residual + RMSNorm input, r = x + b, in the reference's two forms
// (crates/ironmill-inference/src/metal/shaders/norm/superblock_fused_norm.metal:71-123 and norm/fused_residual_norm.metal:54-74):
//   * the fused residual + norm + projection kernel multiplies the UNROUNDED vector: staged value r * gamma (/ awq), the
//     row sums are scaled by rms_inv afterwards (xq_u / meta_u; only when want_u);
//   * every other consumer reads norm_out, the fp16 copy f16(r * rms_inv * gamma): staged value that / awq (xq_r / meta_r;
//     only when want_r), no scaling afterwards.
// Pass 1 loads, forms r (kept in registers: at most kNormChunks chunks of 8 values per thread), writes this CTA's share
// of resid_out = f16(r), stages the unrounded form and sums r^2; the CTA then agrees on rms_inv; pass 2 stages the
// rounded form.  Returns rms_inv (also left in misc[0] for the producer warp).
// mail != nullptr (tensor parallel): operand b is the sum of a mailbox's nsum slots (`slot` pairs apart, one per rank,
// written over NVLink with `tag` beside every pair of values): f32 in rank order, rounded to fp16 (what the
// stand-alone all-reduce hands to the next kernel).  The reads spin until the tags are there.
// One 8-element chunk of the residual sum: r = x + b (b from memory or from the mailbox slots), the chunk's norm weights
// and activation scales as loaded.
__device__ __forceinline__ void norm_load(const __half *__restrict__ x, const __half *b, const __half *__restrict__ gamma,
                                          const __half *__restrict__ awq, int k, const uint2 *mail, int nsum, int slot, unsigned tag, int *err,
                                          unsigned limit_ms, float (&r)[8], uint4 &rgam, uint4 &rawq) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(x + k);
    rgam = *reinterpret_cast<const uint4 *>(gamma + k);
    rawq = make_uint4(0, 0, 0, 0);
    if (awq) rawq = *reinterpret_cast<const uint4 *>(awq + k);
    float v[8], fb[8];
    unpack8(raw, v);
    if (mail) {
#pragma unroll
        for (int i = 0; i < 8; i++) fb[i] = 0.0f;
        for (int rk = 0; rk < nsum; rk += 2) {  // two slots' reads travel together
            const bool two = rk + 1 < nsum;
            const uint4 *s0 = reinterpret_cast<const uint4 *>(mail + (size_t)rk * slot + (k >> 1));
            const uint4 *s1 = two ? reinterpret_cast<const uint4 *>(mail + (size_t)(rk + 1) * slot + (k >> 1)) : s0;
            uint4 a0 = ld_mail(s0), c0 = ld_mail(s0 + 1), a1 = ld_mail(s1), c1 = ld_mail(s1 + 1);
            mail_settle(s0, a0, c0, tag, err, limit_ms);
            mail_settle(s1, a1, c1, tag, err, limit_ms);
            float fr[8];
            unpack2(a0.x, fr[0], fr[1]); unpack2(a0.z, fr[2], fr[3]); unpack2(c0.x, fr[4], fr[5]); unpack2(c0.z, fr[6], fr[7]);
#pragma unroll
            for (int i = 0; i < 8; i++) fb[i] += fr[i];
            if (two) {
                unpack2(a1.x, fr[0], fr[1]); unpack2(a1.z, fr[2], fr[3]); unpack2(c1.x, fr[4], fr[5]); unpack2(c1.z, fr[6], fr[7]);
#pragma unroll
                for (int i = 0; i < 8; i++) fb[i] += fr[i];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++) fb[i] = __half2float(__float2half_rn(fb[i]));
    } else {
        const uint4 rb = __ldcg(reinterpret_cast<const uint4 *>(b + k));
        unpack8(rb, fb);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) r[i] = v[i] + fb[i];
}

__device__ __forceinline__ float mega_stage_norm(const __half *__restrict__ x, const __half *b, const __half *__restrict__ gamma,
                                                 const __half *__restrict__ awq, __half *__restrict__ resid_out, int G, bool want_u,
                                                 uint32_t *xq_u, float2 *meta_u, bool want_r, uint32_t *xq_r, float2 *meta_r, float eps,
                                                 float *misc, const uint2 *mail, int nsum, int slot, unsigned tag, int *err,
                                                 unsigned limit_ms) {
    const int lane = threadIdx.x & 31, hl = lane & 15, warp = threadIdx.x >> 5;
    float sq = 0.0f;
    // the thread's first chunk stays in registers between the passes (hidden sizes up to 4096: its only chunk);
    // further chunks are loaded again in pass 2
    float r0[8];
    uint4 rg0 = make_uint4(0, 0, 0, 0), ra0 = rg0;
#pragma unroll
    for (int i = 0; i < 8; i++) r0[i] = 0.0f;
#pragma unroll 1
    for (int g0 = warp * 2; g0 < G; g0 += kV2Consumers * 2) {
        const int grp = g0 + (lane >> 4);
        const bool live = grp < G;
        const int k = (live ? grp : g0) * 128 + hl * 8;
        float r[8];
        uint4 rg, ra;
        norm_load(x, b, gamma, awq, k, mail, nsum, slot, tag, err, limit_ms, r, rg, ra);
        unsigned hres[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            if (live) sq += r[i] * r[i] + r[i + 1] * r[i + 1];
            hres[i >> 1] = (unsigned)__half_as_ushort(__float2half_rn(r[i])) | ((unsigned)__half_as_ushort(__float2half_rn(r[i + 1])) << 16);
        }
        if (live && resid_out && (unsigned)(grp * 16 + hl) % gridDim.x == blockIdx.x)
            *reinterpret_cast<uint4 *>(resid_out + k) = make_uint4(hres[0], hres[1], hres[2], hres[3]);
        if (g0 == warp * 2) {
#pragma unroll
            for (int i = 0; i < 8; i++) r0[i] = r[i];
            rg0 = rg;
            ra0 = ra;
        }
        if (want_u) {
            float v[8], fg[8], a[8];
            unpack8(rg, fg);
            if (awq) unpack8(ra, a);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                v[i] = r[i] * fg[i];
                if (awq) v[i] = div_awq(v[i], a[i]);
            }
            stage_chunk24<1>(v, live, grp, 0, hl, xq_u, meta_u);
        }
    }
    sq = warp_sum(sq);
    if (lane == 0) misc[8 + warp] = sq;
    consumer_sync();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < kV2Consumers; w++) tot += misc[8 + w];
    const float ri = rsqrtf(tot / (float)(G * 128) + eps);
    if (threadIdx.x == 0) misc[0] = ri;  // reaches the producer warp through the slot releases
    if (want_r) {
#pragma unroll 1
        for (int g0 = warp * 2; g0 < G; g0 += kV2Consumers * 2) {
            const int grp = g0 + (lane >> 4);
            const bool live = grp < G;
            float r[8];
            uint4 rg = rg0, ra = ra0;
            if (g0 == warp * 2) {
#pragma unroll
                for (int i = 0; i < 8; i++) r[i] = r0[i];
            } else {  // hidden sizes above 4096 (never with a mailbox: the engine keeps those on the per-kernel schedule)
                norm_load(x, b, gamma, awq, (live ? grp : g0) * 128 + hl * 8, nullptr, 0, 0, 0u, err, limit_ms, r, rg, ra);
            }
            float v[8], fg[8], a[8];
            unpack8(rg, fg);
            if (awq) unpack8(ra, a);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                v[i] = __half2float(__float2half_rn(r[i] * ri * fg[i]));  // norm_out as the reference stores it
                if (awq) v[i] = div_awq(v[i], a[i]);
            }
            stage_chunk24<1>(v, live, grp, 0, hl, xq_r, meta_r);
        }
    }
    return ri;
}

// The item phases run out of line: they are cold next to the projection loop, and a call boundary keeps their
// register appetite (the encoder holds 64 matrix values in flight) from spilling the loop's state.
// ---- the QJL projection of a head item by all four groups ------------------------------------------------------
// A head item runs on group 0, but its projection reads a 64 KB matrix: alone, a thread brings its column in two
// waves of 64 loads, two trips to L2 on the phase's critical path.  Here every consumer thread holds 32 values of a
// column (rows 32 * group ..., loaded before the barrier that opens the phase: the matrix is a constant), and the
// sum walks k upwards through the four groups in turn, handing the running value on through shared memory, so the
// additions happen in exactly the encoder's order.
struct QjlCoop {
    const float (&sv)[32];
    float *carry;  // [128]
    __device__ __forceinline__ void begin(int, int) {}
    template <bool EXACT>
    __device__ __forceinline__ float step(float acc, const float *vec, int group) const {
#pragma unroll
        for (int j = 0; j < 32; j++)
            acc = EXACT ? __fadd_rn(acc, __fmul_rn(sv[j], vec[32 * group + j])) : fmaf(sv[j], vec[32 * group + j], acc);
        return acc;
    }
    // group 0's side: 1 + kGroups CTA-wide barriers, matched by assist() on the other groups
    template <bool EXACT, class Scope>
    __device__ __forceinline__ float finish(const Scope &, const float *vec, int d, int) {
        consumer_sync();  // vec is visible to every group
        carry[d] = step<EXACT>(0.0f, vec, 0);
#pragma unroll
        for (int gi = 0; gi < kGroups; gi++) consumer_sync();
        return carry[d];
    }
    template <bool EXACT>
    __device__ __forceinline__ void assist(const float *vec, int d, int group) const {
        consumer_sync();
#pragma unroll
        for (int gi = 0; gi < kGroups; gi++) {
            if (gi == group) carry[d] = step<EXACT>(carry[d], vec, group);
            consumer_sync();
        }
    }
};

template <int GQ>
__device__ IM_MEGA_ITEM_INLINE void mega_attention_item(const GroupScope &gs, AttnSmem<GQ> &sm, const float *cbk, const float *cbv, const AttnParams &ap,
                                                 int kvh, int split, int r0, int r1) {
    tq_attention_item<GQ>(gs, sm, cbk, cbv, ap, kvh, 0, split, r0, r1);
}

// Combine the splits of one query head and rotate back, by all 16 consumer warps.  Warp w takes splits w, w + 16, ...:
// a lane loads four output dimensions of up to five splits (and their max / sum) in one trip to L2 and folds them
// under the warp's own running max; group 0 then merges the 16 warp partials and applies the rotation.
__device__ IM_MEGA_ITEM_INLINE void mega_reduce_head(const GroupScope &gs, int group, int tid, float *U, const float *__restrict__ po,
                                              const float *__restrict__ pm, const float *__restrict__ pl, const float *__restrict__ signs,
                                              __half *__restrict__ attn_out, int head, int splits, int used) {
    constexpr int kBatch = 5;
    float *part = U;                                 // [16][128]
    float *part_ml = part + kV2Consumers * kHd;      // [16][2]
    float *xs = part_ml + 2 * kV2Consumers;          // 128 floats for the rotation
    const int warp = tid >> 5, lane = tid & 31;
    const size_t base = (size_t)head * splits;
    float wm = -INFINITY, wl = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s0 = warp; s0 < used; s0 += kV2Consumers * kBatch) {
        float4 o[kBatch];
        float m[kBatch], l[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; j++) {
            const int sp = s0 + j * kV2Consumers;
            const bool live = sp < used;
            o[j] = live ? __ldcg(reinterpret_cast<const float4 *>(po + (base + sp) * kHd) + lane) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            m[j] = live ? __ldcg(pm + base + sp) : -INFINITY;
            l[j] = live ? __ldcg(pl + base + sp) : 0.0f;
        }
        float bm = wm;
#pragma unroll
        for (int j = 0; j < kBatch; j++) bm = fmaxf(bm, m[j]);
        const float c0 = wm == -INFINITY ? 0.0f : __expf(wm - bm);
        acc.x *= c0; acc.y *= c0; acc.z *= c0; acc.w *= c0;
        wl *= c0;
#pragma unroll
        for (int j = 0; j < kBatch; j++) {
            const float c = m[j] == -INFINITY ? 0.0f : __expf(m[j] - bm);
            acc.x = fmaf(o[j].x, c, acc.x); acc.y = fmaf(o[j].y, c, acc.y);
            acc.z = fmaf(o[j].z, c, acc.z); acc.w = fmaf(o[j].w, c, acc.w);
            wl = fmaf(l[j], c, wl);
        }
        wm = bm;
    }
    reinterpret_cast<float4 *>(part + warp * kHd)[lane] = acc;
    if (lane == 0) {
        part_ml[warp * 2] = wm;
        part_ml[warp * 2 + 1] = wl;
    }
    consumer_sync();
    if (group == 0) {
        const int d = tid;
        float gm = -INFINITY;
#pragma unroll
        for (int i = 0; i < kV2Consumers; i++) gm = fmaxf(gm, part_ml[i * 2]);
        float a = 0.0f, lt = 0.0f;
#pragma unroll
        for (int i = 0; i < kV2Consumers; i++) {
            const float m = part_ml[i * 2];
            const float corr = m == -INFINITY ? 0.0f : __expf(m - gm);
            a = fmaf(part[i * kHd + d], corr, a);
            lt = fmaf(part_ml[i * 2 + 1], corr, lt);
        }
        const float r = hadamard_thread(gs, a / fmaxf(lt, 1e-10f), signs[d], xs, kHd);
        attn_out[(size_t)head * kHd + d] = __float2half_rn(r);
    }
    consumer_sync();
}

}  // namespace

// TP: the tensor-parallel variant (exchange of the row-split projections' partial sums between the ranks' kernels);
// compiled apart so that the single-GPU kernel carries none of it.
// BITS: bits per cached element (8 or 4), a compile-time constant so that the cache-format branches of the shared bodies fold away.
template <int GQ, bool TP, int BITS>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_token_kernel(const MegaParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int nring = p.nring;
    unsigned char *ring = smem;
    float *red = reinterpret_cast<float *>(ring + (size_t)nring * kStageBytes);
    float *cbk = red + (size_t)nring * kRedFloats;  // K codebook (128), V codebook (256)
    float *cbv = cbk + 128;
    float *bdk = cbv + 256;                          // suffix-minimum boundary tables of the encoder: K (127), V (255)
    float *bdv = bdk + 128;
    float *misc = bdv + 256;                         // [0] rms_inv, [8..23] reduction scratch, [30] wait result
    // descriptors of the current and the next layer (5 phase blocks per layer: the four projections and the next
    // layer's QKV; plus the layer block), copied one layer ahead so that no phase starts with a global load
    uint32_t *desc = reinterpret_cast<uint32_t *>(misc + 32);   // [2][kDescWords]
    uint64_t *full = reinterpret_cast<uint64_t *>(desc + 2 * kDescWords);
    uint64_t *empty = full + nring;
    unsigned char *U = reinterpret_cast<unsigned char *>(empty + nring);  // phase scratch (16-byte aligned by construction)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NP = 4 * p.L;
    // Patience of every wait.  Tensor parallel: a rank may sit behind a peer whose launch came later (host jitter, a
    // graph being instantiated), and while its consumers wait for that peer its producer waits for them.
    const unsigned wait_ms = p.wait_ms ? p.wait_ms : (TP ? 5000u : (unsigned)(kWaitLimitNs / 1000000ull));
    // tags of this launch's mailbox stores: launch number x 2 L + 2 layer + (o: 1, down: 2); never 0, never repeated
    const unsigned xbase = TP ? (unsigned)ld_volatile(reinterpret_cast<const int *>(p.xepoch)) * (unsigned)(2 * p.L) : 0u;
    // words of layer l's descriptors -> desc[l & 1]; called by consumer threads one layer ahead (and for layer 0 at start)
    auto copy_desc = [&](int l, int t, int nthreads) {
        uint32_t *dst = desc + (l & 1) * kDescWords;
        const uint32_t *src_ph = reinterpret_cast<const uint32_t *>(p.phases + 4 * l);
        const int nph = min(5, NP - 4 * l) * kPhaseWords;
        for (int i = t; i < nph; i += nthreads) dst[i] = src_ph[i];
        const uint32_t *src_ly = reinterpret_cast<const uint32_t *>(p.layers + l);
        for (int i = t; i < kLayerWords; i += nthreads) dst[5 * kPhaseWords + i] = src_ly[i];
    };
    copy_desc(0, tid, kMegaThreads);

    if (tid == 0) {
        for (int i = 0; i < nring; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kV2Consumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (p.trace && blockIdx.x == 0) p.trace[0] = global_ns();
    }
    for (int i = tid; i < 128 + 256; i += kMegaThreads) {
        cbk[i] = i < 128 ? (i < p.k_levels ? p.k_cb[i] : 0.0f) : (i - 128 < p.v_levels ? p.v_cb[i - 128] : 0.0f);
        bdk[i] = i < 128 ? (i < p.k_levels - 1 ? p.k_bd[i] : INFINITY) : (i - 128 < p.v_levels - 1 ? p.v_bd[i - 128] : INFINITY);
    }
    __syncthreads();

    if (warp == kV2Consumers) {
        // =========================================================== producer warp
        // Lane 0 issues the stages of every phase in order.  Before a slot is refilled the warp waits for the
        // consumers to release it; if the stage that lived there ended a row block, the warp adds the sixteen
        // partial sums in warp order, applies the epilogue and writes the outputs; after the last stage of a
        // phase it arrives at that phase's grid barrier.
        struct Cursor {
            int q;          // phase
            StageIter it;
            MegaPhase ph;
        };
        auto open = [&](Cursor &c, int q) {
            c.q = q;
            if (q < NP) {
                c.ph = p.phases[q];
                const Range r = cta_range(c.ph.nblk, c.ph.G);
                c.it = StageIter(r.t_begin, r.t_end, c.ph.G);
            }
        };
        auto arrive = [&](int q, int xout) {  // all lanes' output writes precede the arrival
            if (TP && xout) return;  // the outputs went to every rank with their tags: readers wait on those, not on a count
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(p.bar + phase_barrier(q), 1u);
        };
        Cursor issue{0, StageIter(0, 0, 1), MegaPhase{}}, done{0, StageIter(0, 0, 1), MegaPhase{}};
        open(issue, 0);
        open(done, 0);
        // Phases in which this CTA has no tiles are passed without an arrival from this warp: the CTA's consumers
        // arrive for it once they have staged the phase's input (matvec_phase), so that nobody can overwrite a buffer
        // they still read.
        auto skip_empty_done = [&]() {
            while (done.q < NP && done.it.t >= done.it.t_end) open(done, done.q + 1);
        };
        skip_empty_done();
        bool ok = true;
        auto reclaim = [&](int slot_, int parity) {  // the oldest stage in flight lives in slot_
            if (ok && !mbar_wait_warp(&empty[slot_], parity, p.err, wait_ms)) ok = false;
            int dt0, dn, drb, dgrp;
            done.it.next(dt0, dn, drb, dgrp);
            const MegaPhase &ph = done.ph;
            if (ok && dgrp + dn == ph.G) {  // the stage ended a row block: combine and write
                const float *buf = red + slot_ * kRedFloats;
                float v = 0.0f;
                if (lane < 16) {
#pragma unroll
                    for (int w = 0; w < kV2Consumers; w++) v += buf[w * 16 + lane];
                }
                // rows that multiplied the unrounded vector still need the norm's scale; norm_out carries it already
                const float ri = (ph.resid && drb * 16 < ph.split_row) ? misc[0] : 1.0f;
                const float vu = __shfl_down_sync(0xffffffffu, v, 8);  // lanes 0-7: the up row of the same output
                if (ph.gate_up) {
                    const float gv = v * ri, uv = vu * ri;
                    const int n = drb * 8 + lane;
                    if (lane < 8 && n < ph.N) ph.y[n] = __float2half_rn((gv / (1.0f + expf(-gv))) * uv);
                } else {
                    const int n = drb * 16 + lane;
                    const __half h = __float2half_rn(v * ri);
                    if (TP && ph.xout) {
                        // this rank's partial sums: two outputs and the tag per 8-byte store, one store per rank (its own included)
                        const unsigned mine = (unsigned)__half_as_ushort(h);
                        const unsigned next = __shfl_down_sync(0xffffffffu, mine, 1);
                        if (lane < 16 && !(lane & 1) && n < ph.N) {  // N is a multiple of 16
                            const unsigned tag = xbase + (unsigned)((done.q >> 2) * 2 + ((ph.xout - 1) & 1) + 1);
                            const size_t off = ((size_t)(ph.xout - 1) * p.world + p.rank) * (size_t)(p.xH >> 1) + (size_t)(n >> 1);
                            for (int r = 0; r < p.world; r++)
                                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p.xmail[r] + off), "r"(mine | (next << 16)), "r"(tag) : "memory");
                        }
                    } else if (lane < 16 && n < ph.N) {
                        ph.y[n] = h;
                    }
                }
            }
            if (done.it.t >= done.it.t_end) {  // that was this CTA's last stage of the phase
                arrive(done.q, done.ph.xout);
                open(done, done.q + 1);
                skip_empty_done();
            }
        };
        int slot = 0, phase = 0, nstages = 0;
        int t0, n, rb0, grp0;
        while (issue.q < NP) {
            if (!issue.it.next(t0, n, rb0, grp0)) {
                open(issue, issue.q + 1);
                continue;
            }
            if (nstages >= nring) reclaim(slot, phase ^ 1);
            if (lane == 0) {
                mbar_expect_tx(&full[slot], (uint32_t)(n * kTileBytes));
                bulk_g2s(ring + (size_t)slot * kStageBytes, issue.ph.tiles + (size_t)t0 * kTileBytes, (uint32_t)(n * kTileBytes), &full[slot]);
            }
            nstages++;
            if (++slot == nring) {
                slot = 0;
                phase ^= 1;
            }
        }
        int left = nstages < nring ? nstages : nring;
        int dslot = nstages < nring ? 0 : slot, dphase = nstages < nring ? 0 : (phase ^ 1);
        for (; left > 0; left--) {
            reclaim(dslot, dphase);
            if (++dslot == nring) {
                dslot = 0;
                dphase ^= 1;
            }
        }
    } else {
        // =========================================================== consumers
        // staged activations of up to g_cap groups: two fix-up constants per group, then three byte planes of 32 words.
        // The QKV phases of layers >= 1 stage a second set (their K and V rows read the fp16 norm_out while the Q rows read
        // the unrounded vector, mega_stage_norm): it starts g_norm groups into the same arrays (g_cap >= 2 g_norm).
        float2 *meta = reinterpret_cast<float2 *>(U);                                      // [g_cap][2]
        uint32_t *xq = reinterpret_cast<uint32_t *>(U + (size_t)p.g_cap * 16);             // [g_cap][3][32] words
        float2 *meta2 = meta + 2 * p.g_norm;
        uint32_t *xq2 = xq + (size_t)p.g_norm * 96;
        const int group = warp >> 2;
        const GroupScope gs{tid & 127, 128, 2 + group};
        bool dead = false;
        int slot = 0, par = 0;

        auto grid_wait = [&](int k) {
            if (tid == 0) {
                const bool okw = dead ? false : grid_poll(p.bar, k, p.err, wait_ms);
                reinterpret_cast<int *>(misc)[30] = okw ? 1 : 0;
                if (p.trace && blockIdx.x == 0) p.trace[k + 1] = global_ns();
            }
            consumer_sync();
            if (reinterpret_cast<int *>(misc)[30] == 0) dead = true;
        };
        constexpr bool tp = TP;
        // Tensor parallel: no barrier follows a row-split projection (the next phase's staging waits on the tags of
        // the values it reads); CTA 0 still leaves its stamp so that the phase accounting keeps its seven columns.
        auto xrank_wait = [&](int k, int) {
            if (tid == 0 && p.trace && blockIdx.x == 0) p.trace[k + 1] = global_ns();
        };
        auto items_done = [&](int k) {  // every consumer thread has finished its items of the phase
            consumer_sync();
            if (tid == 0) grid_arrive(p.bar, k);
        };

        const int g = lane >> 2, t = lane & 3;
        TileMath<1, false> tm;
        tm.reset();

        // One projection: stage the activations, then walk this CTA's stages of the phase.
        auto matvec_phase = [&](int q) __attribute__((always_inline)) {
            const MegaPhase ph = *reinterpret_cast<const MegaPhase *>(desc + ((q >> 2) & 1) * kDescWords + (q & 3) * kPhaseWords);
            const int G = ph.G;
            const Range r = cta_range(ph.nblk, G);
            if (ph.resid) {
                // tensor parallel: gate/up reads this layer's o sums, QKV the previous layer's down sums
                const bool from_mail = TP && ph.xin;
                const uint2 *mail = from_mail ? p.xmail[p.rank] + (size_t)(ph.xin - 1) * p.world * (size_t)(p.xH >> 1) : nullptr;
                const unsigned tag = xbase + (unsigned)((((q & 3) == 0 ? (q >> 2) - 1 : (q >> 2)) * 2) + ((ph.xin - 1) & 1) + 1);
                // rows below split_row multiply the unrounded vector (primary set), the others norm_out (the second set, or
                // the primary one when no row of the phase wants the unrounded vector).  A CTA stages only the sets its own
                // row blocks read: with whole row blocks per CTA almost every CTA of a QKV phase needs just one of them.
                const bool phase_u = ph.split_row > 0;
                const bool want_u = phase_u && r.t_begin < r.t_end && (r.t_begin / G) * 16 < ph.split_row;
                const bool want_r = r.t_begin < r.t_end && (r.t_end / G) * 16 > ph.split_row;
                mega_stage_norm(ph.x, ph.resid, ph.gamma, ph.awq, ph.resid_out, G, want_u, xq, meta, want_r, phase_u ? xq2 : xq,
                                phase_u ? meta2 : meta, p.eps, misc, mail, p.world, p.xH >> 1, tag, p.err, wait_ms);
            } else {
                mega_stage_plain(ph.x, ph.awq, G, xq, meta);
            }
            consumer_sync();
            // A CTA without tiles in this phase arrives at its barrier here, after every consumer thread has read the
            // phase's input (a CTA with tiles arrives from its producer warp, after its last stage was released).
            if (r.t_begin >= r.t_end && tid == 0 && !(TP && ph.xout)) grid_arrive(p.bar, phase_barrier(q));
            if (q + 1 < NP) {  // the next projection's activation scales and norm weight: one pass through a 4.9 GB weight
                               // stream evicts them from L2 every token, so ask for them now, one 128-byte line per thread
                const MegaPhase nx = *reinterpret_cast<const MegaPhase *>(desc + ((q >> 2) & 1) * kDescWords + ((q & 3) + 1) * kPhaseWords);
                for (int i = blockIdx.x + gridDim.x * tid; i < 2 * nx.G; i += gridDim.x * kV2Consumers * 32) {
                    if (nx.awq) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx.awq + i * 64));
                    if (nx.gamma) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx.gamma + i * 64));
                }
            }
            tm.reset();
            const bool two_sets = ph.resid && ph.split_row > 0 && ph.split_row < ph.N;
            // This CTA's row blocks, each a run of stages of up to kStageTiles tiles (the same walk as the producer's StageIter,
            // written as two plain loops: the iterator's arithmetic per stage cost 15 % of the loop's time).
            const int rb_end = r.t_end / G;
            for (int rb = r.t_begin / G; rb < rb_end; rb++) {
                const bool sec = two_sets && rb * 16 >= ph.split_row;  // this row block reads norm_out
                const uint32_t *xq_rb = sec ? xq2 : xq;
                const float2 *meta_rb = sec ? meta2 : meta;
                for (int grp0 = 0; grp0 < G; grp0 += kStageTiles) {
                    const int n = min(kStageTiles, G - grp0);
                    if (!dead && !mbar_wait_warp(&full[slot], par, p.err, wait_ms)) dead = true;
                    const unsigned char *st = ring + (size_t)slot * kStageBytes;
                    if (!dead && warp < n) {
                        const int tb = warp + kV2Consumers;
                        tm.pair(st + (size_t)warp * kTileBytes, grp0 + warp, st + (size_t)tb * kTileBytes, grp0 + tb, tb < n, xq_rb, meta_rb, lane);
                    }
                    if (grp0 + n == G) {  // last stage of the row block: hand the partial sums to the producer warp
                        float *buf = red + slot * kRedFloats;
                        float r0, r1;
                        tm.row_sums(0, r0, r1);
                        if (t == 0) {
                            buf[warp * 16 + g] = r0;
                            buf[warp * 16 + g + 8] = r1;
                        }
                        tm.clear_sums();
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[slot]);
                    if (++slot == nring) {
                        slot = 0;
                        par ^= 1;
                    }
                }
            }
        };

        const int seq_len = min(p.pos[0] + 1, p.max_seq);  // the host checks the position before every step; never read past the caches
        int chunk = (seq_len + p.splits - 1) / p.splits;
        chunk = (chunk + kTile - 1) / kTile * kTile;
        const int used = (seq_len + chunk - 1) / chunk;  // splits that hold positions (<= p.splits)

        const int n_heads = p.nh + 2 * p.nkv;
        for (int l = 0; l < p.L; l++) {
            const MegaLayer ly = *reinterpret_cast<const MegaLayer *>(desc + (l & 1) * kDescWords + 5 * kPhaseWords);
            // ---- QKV (layer 0: plain, on the normalised embedding; later layers: residual + norm prologue)
            if (l > 0) {  // the previous layer's down projection
                if (tp) xrank_wait(7 * l - 1, 2 * (l - 1) + 1); else grid_wait(7 * l - 1);
            }
            matvec_phase(4 * l);
            float sv[32];  // this thread's share of the projection matrix, on its way while the grid gathers
            if (blockIdx.x < n_heads) {
#pragma unroll
                for (int j = 0; j < 32; j++) sv[j] = __ldg(p.qjl_t + (size_t)(32 * group + j) * kHd + gs.d);
            }
            grid_wait(7 * l);
            // the next layer's descriptors: the buffer's previous tenant (layer l - 1) was last read before the barrier above
            // (by the threads of groups 1-3: group 0 carries the head items of the phase that starts here)
            if (l + 1 < p.L && tid >= 128) copy_desc(l + 1, tid - 128, kV2Consumers * 32 - 128);

            // ---- (QK-norm,) RoPE, cache write, query rotation: one head per 128-thread group
            {
                PrepArgs a;
                a.qkv = p.qkv; a.stride = p.q_dim + 2 * p.kv_dim; a.k_off = p.q_dim; a.v_off = p.q_dim + p.kv_dim; a.kv = nullptr; a.kv_stride = 0;
                a.qw = ly.q_norm; a.kw = ly.k_norm; a.cosc = p.cosc; a.sinc = p.sinc;
                a.nh = p.nh; a.nkv = p.nkv; a.rotary_dim = p.rotary_dim; a.with_norm = p.with_qk_norm; a.T = 1; a.max_seq = p.max_seq;
                a.base_pos = seq_len - 1; a.eps = p.eps; a.pos_dev = nullptr; a.slot_map = nullptr; a.qrot = p.qrot; a.q_out = nullptr;  // the position was read once at the start
                a.ktab = EncodeTables{p.signs, cbk, bdk, p.qjl_t, p.k_levels, 1, BITS};
                a.vtab = EncodeTables{p.signs, cbv, bdv, p.qjl_t, p.v_levels, 0, BITS};
                a.kc = ly.kc; a.vc = ly.vc; a.ks = ly.ks; a.vs = ly.vs; a.krn = ly.krn; a.no_q_proj = 0;
                float *sh = reinterpret_cast<float *>(U);
                QjlCoop pj{sv, sh + 3 * kHd + 4};
                if (!dead)
                    for (int item = blockIdx.x; item < n_heads; item += gridDim.x) {
                        if (group == 0)
                            tq_prep_item(gs, a, sh, item, 0, pj);
                        else if (item < p.nh)
                            pj.assist<false>(sh, gs.d, group);            // query head: projects the rotated query
                        else if (item < p.nh + p.nkv)
                            pj.assist<true>(sh + 2 * kHd, gs.d, group);  // key head: projects the residual
                    }
            }
            items_done(7 * l + 1);
            // This group's first attention item: its cached rows do not depend on this layer's cache write (only the row
            // of the token being decoded does), so L2 is asked for them before the barrier (no registers held across it).
            AttnParams ap;
            ap.q = nullptr; ap.kc = ly.kc; ap.vc = ly.vc; ap.ks = ly.ks; ap.vs = ly.vs; ap.krn = ly.krn;
            ap.signs = p.signs; ap.qjl = p.qjl_t; ap.k_cb = p.k_cb; ap.v_cb = p.v_cb; ap.qrot = p.qrot;
            ap.po = p.po; ap.pm = p.pm; ap.pl = p.pl; ap.attn_scale = p.attn_scale; ap.qjl_factor = p.qjl_factor;
            ap.nh = p.nh; ap.nkv = p.nkv; ap.max_seq = p.max_seq; ap.base_pos = 0; ap.T = 1; ap.splits = p.splits; ap.pos_dev = p.pos; ap.slot_map = nullptr; ap.bits = BITS;
            const int item0 = blockIdx.x + gridDim.x * group;
            const bool have0 = !dead && item0 < p.nkv * used;
            if (have0) {
                const int split = item0 / p.nkv;
                tq_attention_l2_prefetch(gs.d, ap, item0 % p.nkv, 0, split * chunk, min(split * chunk + chunk, seq_len), seq_len - 1);
            }
            grid_wait(7 * l + 1);

            // ---- split attention: one (KV head, split) per group
            {
                AttnSmem<GQ> &sm = reinterpret_cast<AttnSmem<GQ> *>(U)[group];
                if (!dead)
                    for (int item = item0; item < p.nkv * used; item += gridDim.x * kGroups) {
                        const int kvh = item % p.nkv, split = item / p.nkv;
                        mega_attention_item<GQ>(gs, sm, cbk, cbv, ap, kvh, split, split * chunk, min(split * chunk + chunk, seq_len));
                    }
            }
            items_done(7 * l + 2);
            grid_wait(7 * l + 2);

            // ---- combine the splits, rotate back: one query head per CTA.  The four groups each combine a quarter
            // of the splits (their loads all in flight together), group 0 merges the four and rotates back.
            if (!dead)
                for (int head = blockIdx.x; head < p.nh; head += gridDim.x)
                    mega_reduce_head(gs, group, tid, reinterpret_cast<float *>(U), p.po, p.pm, p.pl, p.signs, p.attn_out, head, p.splits, used);
            items_done(7 * l + 3);
            grid_wait(7 * l + 3);

            matvec_phase(4 * l + 1);  // o
            if (tp) xrank_wait(7 * l + 4, 2 * l); else grid_wait(7 * l + 4);
            matvec_phase(4 * l + 2);  // residual + norm -> gate/up + SiLU
            grid_wait(7 * l + 5);
            matvec_phase(4 * l + 3);  // down
        }
    }

    // ---- exit: the last CTA to leave clears the counters for the next launch
    __syncthreads();
    if (tid == 0) {
        const int nbar = 7 * p.L;
        __threadfence();
        if (atomicAdd(p.bar + nbar, 1u) == gridDim.x - 1) {
            // every CTA has passed every barrier except possibly the very last one (down of the last layer),
            // whose arrivals all precede the exits counted above
            for (int i = 0; i <= nbar; i++) p.bar[i] = 0;
            if (TP) *p.xepoch = *p.xepoch + 1u;  // every CTA read it at its start, long before the last one leaves
            if (p.trace) p.trace[nbar + 1] = global_ns();
        }
    }
}

size_t mega_smem_bytes(int nring, int u_bytes) {
    return (size_t)nring * (kStageBytes + kRedFloats * 4 + 16) + (2 * (128 + 256) + 32) * 4 + 2 * kDescWords * 4 + (size_t)u_bytes;
}

template <int GQ>
static constexpr int attn_bytes() {
    return kGroups * (int)sizeof(AttnSmem<GQ>);
}

int mega_g_cap(int G_max, int G_norm) { return G_max > 2 * G_norm ? G_max : 2 * G_norm; }

int mega_u_bytes(int G_max, int G_norm, int gq) {
    const int stage = mega_g_cap(G_max, G_norm) * (16 + 3 * 32 * 4);
    int attn = 0;
    switch (gq) {
        case 1: attn = attn_bytes<1>(); break;
        case 2: attn = attn_bytes<2>(); break;
        case 4: attn = attn_bytes<4>(); break;
        case 8: attn = attn_bytes<8>(); break;
        default: return -1;
    }
    const int prep = kGroups * (3 * kHd + 4) * 4;
    int u = stage > attn ? stage : attn;
    if (prep > u) u = prep;
    return (u + 15) & ~15;
}

template <int GQ, bool TP, int BITS>
static int mega_launch_t(const MegaParams &p, const Device *dev, cudaStream_t st) {
    const size_t smem = mega_smem_bytes(p.nring, p.u_bytes);
    if (smem > dev->smem_optin) return IM_ERR_BOUNDS;
    auto kern = decode_token_kernel<GQ, TP, BITS>;
    static DeviceOnce once;  // per instantiation
    if (once.first(dev->ordinal)) IM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev->smem_optin));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(dev->sm_count);
    cfg.blockDim = dim3(kMegaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident: the grid barriers need it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    IM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, p));
    return IM_OK;
}

int mega_launch(const MegaParams &p, const Device *dev, cudaStream_t st) {
    if (p.nkv <= 0 || p.nh % p.nkv != 0) return IM_ERR_BOUNDS;
    const bool tp = p.tagged != 0;
    if (p.tq_bits == 4) {  // the 4-bit cache is built for the single-GPU (barrier) form of the kernel
        if (tp) return IM_ERR_BOUNDS;
        switch (p.nh / p.nkv) {
            case 1: return mega_launch_t<1, false, 4>(p, dev, st);
            case 2: return mega_launch_t<2, false, 4>(p, dev, st);
            case 4: return mega_launch_t<4, false, 4>(p, dev, st);
            case 8: return mega_launch_t<8, false, 4>(p, dev, st);
            default: return IM_ERR_BOUNDS;
        }
    }
    switch (p.nh / p.nkv) {
        case 1: return tp ? mega_launch_t<1, true, 8>(p, dev, st) : mega_launch_t<1, false, 8>(p, dev, st);
        case 2: return tp ? mega_launch_t<2, true, 8>(p, dev, st) : mega_launch_t<2, false, 8>(p, dev, st);
        case 4: return tp ? mega_launch_t<4, true, 8>(p, dev, st) : mega_launch_t<4, false, 8>(p, dev, st);
        case 8: return tp ? mega_launch_t<8, true, 8>(p, dev, st) : mega_launch_t<8, false, 8>(p, dev, st);
        default: return IM_ERR_BOUNDS;
    }
}

}  // namespace im
