// Building blocks of the tiled INT4 matvec shared by the stand-alone kernel and the whole-token decode kernel:
// mbarrier / bulk-copy wrappers with bounded waits, the u8 x s8 tensor-core instruction, the stage iterator.
#pragma once
#include "common.cuh"

namespace im {

constexpr int kV2Consumers = 16;
constexpr int kV2Threads = (kV2Consumers + 1) * 32;
constexpr int kTileCodeBytes = 1024;
constexpr int kTileBytes = 1088;     // 1024 bytes of nibbles + 16 (scale, zero) fp16 pairs, contiguous
constexpr int kStageTiles = 32;      // tiles per stage: two per consumer warp
constexpr unsigned long long kWaitLimitNs = 400ull * 1000 * 1000;  // bounded mbarrier waits: give up, flag, carry on without computing

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false (and the error word set) if the barrier never completed.
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// limit_ms: patience of this wait (default: kWaitLimitNs); a kernel that may legitimately sit behind another GPU passes more
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err, unsigned limit_ms = (unsigned)(kWaitLimitNs / 1000000ull)) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned i = 1;; i++) {
        __nanosleep(32);  // back off: a tight poll from many threads competes with the bulk copies for shared memory
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 0 && global_ns() - t0 > (unsigned long long)limit_ms * 1000000ull) break;
    }
    atomicExch(err, 1);
    return false;
}
// One lane polls for the warp.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, int *err, unsigned limit_ms = (unsigned)(kWaitLimitNs / 1000000ull)) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, err, limit_ms) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// First product of an accumulator: C = 0 comes from the zero register, no moves to clear it.
__device__ __forceinline__ void mma_u8s8_z(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// The arithmetic of the consumer warps: two tiles (16 rows x 128 columns of 4-bit codes each) against the staged
// activations of their groups, then the per-(row, group) float fix-up  s * sx * (sum_k xi_k q_k - z * sum_k xi_k)
// (with meta = (sx / 16, 16 * sum_k xi_k): the integer dot product arrives multiplied by 16, see pair()).
// Lane (g = lane >> 2, t = lane & 3) holds rows g and g + 8 of batch row t in acc0 / acc1.
// The activation fragments of a group stay in registers until the warp is handed another group: with K = 4096 a
// stage is a whole row block, every warp sees the same two groups stage after stage, and the fragments are read
// from shared memory once per projection.
template <int NB>
struct TileMath {
    uint4 xa0, xa1, xb0, xb1;  // B fragments of the groups ga / gb (words of columns 2b = high bytes, 2b + 1 = low bytes)
    int ga, gb;
    float acc0, acc1;
    __device__ __forceinline__ void reset() {  // new activations were staged
        ga = gb = -1;
        acc0 = acc1 = 0.0f;
        xa0 = xa1 = xb0 = xb1 = make_uint4(0, 0, 0, 0);
    }
    // xq words: index ((grp*2NB + col)*4 + t)*8 ..; meta[grp*NB + b] = (scale, sum of the 128 integers)
    __device__ __forceinline__ void pair(const unsigned char *tile_a, int grp_a, const unsigned char *tile_b, int grp_b, bool have_b,
                                         const uint32_t *xq, const float2 *meta, int lane) {
        const int g = lane >> 2, t = lane & 3;
        const uint4 a0 = *reinterpret_cast<const uint4 *>(tile_a + lane * 16);        // row g
        const uint4 a1 = *reinterpret_cast<const uint4 *>(tile_a + 512 + lane * 16);  // row g + 8
        uint4 b0 = make_uint4(0, 0, 0, 0), b1 = b0;
        if (have_b) {
            b0 = *reinterpret_cast<const uint4 *>(tile_b + lane * 16);
            b1 = *reinterpret_cast<const uint4 *>(tile_b + 512 + lane * 16);
        }
        if (grp_a != ga) {  // warp-uniform
            ga = grp_a;
            if (g < 2 * NB) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xq + (((size_t)grp_a * 2 * NB + g) * 4 + t) * 8);
                xa0 = xp[0];
                xa1 = xp[1];
            }
        }
        if (have_b && grp_b != gb) {
            gb = grp_b;
            if (g < 2 * NB) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xq + (((size_t)grp_b * 2 * NB + g) * 4 + t) * 8);
                xb0 = xp[0];
                xb1 = xp[1];
            }
        }
        // Low and high nibbles go to separate accumulators: the low ones masked in place, the high ones masked in place
        // too (a byte 16 q, still a valid u8), so a word costs two logic operations and no shift.  The two chains are
        // independent; the fix-up adds them as 16 * low + high16, and the staged activation scale carries the 1/16.
        // B columns of a group: words (even positions, odd positions) of each 8-byte chunk: the low nibbles of a code
        // word are the even columns, the high nibbles the odd ones.
        int cal[4], cah[4], cbl[4], cbh[4];
        constexpr unsigned ML = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
        mma_u8s8_z(cal, a0.x & ML, a1.x & ML, a0.y & ML, a1.y & ML, xa0.x, xa0.z);
        mma_u8s8_z(cbl, b0.x & ML, b1.x & ML, b0.y & ML, b1.y & ML, xb0.x, xb0.z);
        mma_u8s8_z(cah, a0.x & MH, a1.x & MH, a0.y & MH, a1.y & MH, xa0.y, xa0.w);
        mma_u8s8_z(cbh, b0.x & MH, b1.x & MH, b0.y & MH, b1.y & MH, xb0.y, xb0.w);
        mma_u8s8(cal, a0.z & ML, a1.z & ML, a0.w & ML, a1.w & ML, xa1.x, xa1.z);
        mma_u8s8(cbl, b0.z & ML, b1.z & ML, b0.w & ML, b1.w & ML, xb1.x, xb1.z);
        mma_u8s8(cah, a0.z & MH, a1.z & MH, a0.w & MH, a1.w & MH, xa1.y, xa1.w);
        mma_u8s8(cbh, b0.z & MH, b1.z & MH, b0.w & MH, b1.w & MH, xb1.y, xb1.w);
        if (t < NB) {
            {
                const float2 m = meta[grp_a * NB + t];
                const __half2 *szp = reinterpret_cast<const __half2 *>(tile_a + kTileCodeBytes);
                const float2 sz0 = __half22float2(szp[g]), sz1 = __half22float2(szp[g + 8]);
                const float f0 = (float)(cal[0] * 4096 + (cal[1] * 16 + (cah[0] * 256 + cah[1]))), f1 = (float)(cal[2] * 4096 + (cal[3] * 16 + (cah[2] * 256 + cah[3])));
                acc0 = fmaf(sz0.x * m.x, fmaf(-sz0.y, m.y, f0), acc0);
                acc1 = fmaf(sz1.x * m.x, fmaf(-sz1.y, m.y, f1), acc1);
            }
            if (have_b) {
                const float2 m = meta[grp_b * NB + t];
                const __half2 *szp = reinterpret_cast<const __half2 *>(tile_b + kTileCodeBytes);
                const float2 sz0 = __half22float2(szp[g]), sz1 = __half22float2(szp[g + 8]);
                const float f0 = (float)(cbl[0] * 4096 + (cbl[1] * 16 + (cbh[0] * 256 + cbh[1]))), f1 = (float)(cbl[2] * 4096 + (cbl[3] * 16 + (cbh[2] * 256 + cbh[3])));
                acc0 = fmaf(sz0.x * m.x, fmaf(-sz0.y, m.y, f0), acc0);
                acc1 = fmaf(sz1.x * m.x, fmaf(-sz1.y, m.y, f1), acc1);
            }
        }
    }
};

// The same arithmetic on a STRIP: SG = 4 / NB consecutive tiles (groups grp0 .. grp0 + SG - 1) of one row block,
// walked by one warp with ONE pair of accumulators.  An m16n8k32 product has eight B columns and a tile needs only
// 2 NB of them (high and low activation bytes per batch row), so tile j of the strip puts its activations in columns
// 2 NB j .. 2 NB j + 2 NB - 1 and zeros elsewhere: the accumulator then holds the integer dot products of SG different
// (row, group) pairs side by side, every lane owns one of them (rows g and g + 8 of group grp0 + t / NB, batch row
// t % NB), and the float fix-up runs once per strip with all 32 lanes busy instead of once per tile with 8 NB of them.
// A lane feeds column g = lane >> 2: it reads its fragment of the staged activations for the one tile of the strip
// whose columns it owns and a block of zeros for the others (an address select, no register copies).
// acc0 / acc1: this lane's share of rows g / g + 8 (batch row t % NB); row_sums() folds the lanes of a row together.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
template <int NB>
struct StripMath {
    static constexpr int SG = 4 / NB;
    float acc0, acc1;
    __device__ __forceinline__ void reset() { acc0 = acc1 = 0.0f; }
    // tiles: shared-memory address of the strip's first tile; ntiles (1 .. SG, warp-uniform) tiles are present;
    // xq / meta: the staged activations (layout of v2_stage_x); zero32: 32 bytes of zeros in shared memory.
    __device__ __forceinline__ void strip(uint32_t tiles, int grp0, int ntiles, uint32_t xq, const float2 *meta, uint32_t zero32, int lane) {
        const int g = lane >> 2, t = lane & 3;
        const int jm = g / (2 * NB), col = g % (2 * NB);
        const uint32_t xmine = xq + (uint32_t)(((((grp0 + jm) * 2 * NB + col) * 4 + t) * 8) * 4);
        constexpr unsigned ML = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
        int cal[4], cah[4];
#pragma unroll
        for (int j = 0; j < SG; j++) {
            if (j < ntiles) {
                const uint32_t tl = tiles + (uint32_t)(j * kTileBytes + lane * 16);
                const uint4 a0 = lds128(tl), a1 = lds128(tl + 512);
                const uint32_t xp = jm == j ? xmine : zero32;
                const uint4 x0 = lds128(xp), x1 = lds128(xp + 16);
                if (j == 0) {
                    mma_u8s8_z(cal, a0.x & ML, a1.x & ML, a0.y & ML, a1.y & ML, x0.x, x0.z);
                    mma_u8s8_z(cah, a0.x & MH, a1.x & MH, a0.y & MH, a1.y & MH, x0.y, x0.w);
                } else {
                    mma_u8s8(cal, a0.x & ML, a1.x & ML, a0.y & ML, a1.y & ML, x0.x, x0.z);
                    mma_u8s8(cah, a0.x & MH, a1.x & MH, a0.y & MH, a1.y & MH, x0.y, x0.w);
                }
                mma_u8s8(cal, a0.z & ML, a1.z & ML, a0.w & ML, a1.w & ML, x1.x, x1.z);
                mma_u8s8(cah, a0.z & MH, a1.z & MH, a0.w & MH, a1.w & MH, x1.y, x1.w);
            }
        }
        const int jt = t / NB;
        if (jt < ntiles) {
            const float2 m = meta[(grp0 + jt) * NB + t % NB];
            uint32_t s0, s1;
            const uint32_t sza = tiles + (uint32_t)(jt * kTileBytes + kTileCodeBytes + g * 4);
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(s0) : "r"(sza));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(s1) : "r"(sza + 32));
            const float2 sz0 = __half22float2(*reinterpret_cast<const __half2 *>(&s0)), sz1 = __half22float2(*reinterpret_cast<const __half2 *>(&s1));
            const float f0 = (float)(cal[0] * 4096 + (cal[1] * 16 + (cah[0] * 256 + cah[1]))), f1 = (float)(cal[2] * 4096 + (cal[3] * 16 + (cah[2] * 256 + cah[3])));
            acc0 = fmaf(sz0.x * m.x, fmaf(-sz0.y, m.y, f0), acc0);
            acc1 = fmaf(sz1.x * m.x, fmaf(-sz1.y, m.y, f1), acc1);
        }
    }
    // Sums of rows g and g + 8 for batch row t % NB over the lanes that shared them; valid in every lane afterwards.
    __device__ __forceinline__ void row_sums(float &r0, float &r1) const {
        r0 = acc0;
        r1 = acc1;
        if (NB <= 2) {
            r0 += __shfl_xor_sync(0xffffffffu, r0, 2);
            r1 += __shfl_xor_sync(0xffffffffu, r1, 2);
        }
        if (NB == 1) {
            r0 += __shfl_xor_sync(0xffffffffu, r0, 1);
            r1 += __shfl_xor_sync(0xffffffffu, r1, 1);
        }
    }
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kV2Consumers * 32) : "memory"); }

__device__ __forceinline__ unsigned pack4s(int a, int b, int c, int d) {
    return (unsigned)(a & 0xff) | ((unsigned)(b & 0xff) << 8) | ((unsigned)(c & 0xff) << 16) | ((unsigned)(d & 0xff) << 24);
}

struct StageIter {  // 32-bit and division-free in the loop: a 64-bit divide costs more than a tile
    int t, t_end, G, rb, grp;
    __device__ StageIter(int t_begin, int t_end_, int G_) : t(t_begin), t_end(t_end_), G(G_), rb(t_begin / G_), grp(t_begin % G_) {}
    __device__ bool next(int &t0, int &n, int &rb0, int &grp0) {
        if (t >= t_end) return false;
        n = min(min(kStageTiles, G - grp), t_end - t);
        t0 = t;
        rb0 = rb;
        grp0 = grp;
        t += n;
        grp += n;
        if (grp == G) {
            grp = 0;
            rb++;
        }
        return true;
    }
};

}  // namespace im
