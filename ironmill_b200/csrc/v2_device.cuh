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
// 8-bit codes: a tile is 16 rows x 128 columns = 2048 bytes of codes + the same 16 (scale, zero) pairs; a stage holds one
// tile per consumer warp (about the same bytes as a 4-bit stage).
template <int BITS>
struct TileGeom {
    static constexpr int kCodeBytes = BITS == 4 ? im::kTileCodeBytes : 2048;
    static constexpr int kTileBytes = kCodeBytes + 64;
    static constexpr int kStageTiles = BITS == 4 ? im::kStageTiles : kV2Consumers;
};
static_assert(TileGeom<4>::kTileBytes == 1088 && TileGeom<8>::kTileBytes == 2112, "tile_bytes_of (common.cuh) states these sizes");
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
// activations of their groups, then the per-(row, group) float fix-up.
//
// Activations are staged once per CTA as 24-bit integers per group of 128 (xi = round(x * 8355711 / amax), so that all
// three signed bytes of xi stay in [-127, 127]): the rounding is at the level of f32 arithmetic itself, the integer dot
// products are exact.  A batch row occupies four B columns of the m16n8k32 product: high, middle, low byte and a zero
// column; up to two batch rows share a product (eight columns), four batch rows take two.  In the accumulator, lane
// (g = lane >> 2, t = lane & 3) holds rows g and g + 8 of columns 2t and 2t + 1: even t = (high, middle) bytes of batch
// row t / 2, odd t = (low byte, zero).  Both kinds of lane run the same fix-up
//     acc += s * m.x * (256 * v_first + v_second - z * m.y),     v = 16 * (low-nibble sum) + (high-nibble sum as 16 q)
// with their own staged constants m = meta[(group * NB + batch row) * 2 + (t & 1)]:
//     even: (sx * 16, sum(xi) / 16)     odd: (sx / 4096, 0)           (sx = amax / 8355711)
// which add up to s * sx * (sum_k xi_k q_k - z * sum_k xi_k).  row_sums() folds the two lanes of a batch row together.
// The activation fragments of a group stay in registers until the warp is handed another group: with K = 4096 a
// stage is a whole row block, every warp sees the same two groups stage after stage, and the fragments are read
// from shared memory once per projection.
// Staged layout: xq words, index ((grp * 3 NB + 3 b + c) * 4 + t) * 8 + j * 2 + eo, byte plane c = 0 high, 1 middle, 2 low.
constexpr int kActTop = 8355711;  // 0x7F7F7F: the largest staged magnitude
// CACHE = false reads the fragments from shared memory for every pair of tiles instead (four 128-bit loads): 18 registers
// fewer live across the stage loop, which is what the whole-token kernel, at its 96-register ceiling, needs more.
template <int NB, bool CACHE = true>
struct TileMath {
    static constexpr int kSets = (NB + 1) / 2;  // column sets of up to two batch rows
    uint4 xa0[kSets], xa1[kSets], xb0[kSets], xb1[kSets];  // B fragments of the groups ga / gb
    int ga, gb;
    float acc0[kSets], acc1[kSets];
    __device__ __forceinline__ void reset() {  // new activations were staged
        ga = gb = -1;
#pragma unroll
        for (int s = 0; s < kSets; s++) {
            acc0[s] = acc1[s] = 0.0f;
            xa0[s] = xa1[s] = xb0[s] = xb1[s] = make_uint4(0, 0, 0, 0);
        }
    }
    __device__ __forceinline__ void clear_sums() {
#pragma unroll
        for (int s = 0; s < kSets; s++) acc0[s] = acc1[s] = 0.0f;
    }
    __device__ __forceinline__ void load_frag(const uint32_t *xq, int grp, int g, int t, uint4 (&x0)[kSets], uint4 (&x1)[kSets]) {
#pragma unroll
        for (int s = 0; s < kSets; s++) {
            const int b = 2 * s + (g >> 2), c = g & 3;  // this lane's column: byte plane c of batch row b (c = 3: the zero column)
            if (c < 3 && b < NB) {
                const uint4 *xp = reinterpret_cast<const uint4 *>(xq + (((size_t)grp * 3 * NB + 3 * b + c) * 4 + t) * 8);
                x0[s] = xp[0];
                x1[s] = xp[1];
            }
        }
    }
    __device__ __forceinline__ void fix_up(const int (&cl)[4], const int (&ch)[4], const unsigned char *tile, int grp, const float2 *meta,
                                           int s, int g, int t) {
        const int b = 2 * s + (t >> 1);
        if (b < NB) {
            const float2 m = meta[(grp * NB + b) * 2 + (t & 1)];
            const __half2 *szp = reinterpret_cast<const __half2 *>(tile + kTileCodeBytes);
            const float2 sz0 = __half22float2(szp[g]), sz1 = __half22float2(szp[g + 8]);
            const float f0 = fmaf((float)(cl[0] * 16 + ch[0]), 256.0f, (float)(cl[1] * 16 + ch[1]));
            const float f1 = fmaf((float)(cl[2] * 16 + ch[2]), 256.0f, (float)(cl[3] * 16 + ch[3]));
            acc0[s] = fmaf(sz0.x * m.x, fmaf(-sz0.y, m.y, f0), acc0[s]);
            acc1[s] = fmaf(sz1.x * m.x, fmaf(-sz1.y, m.y, f1), acc1[s]);
        }
    }
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
        uint4 la0[kSets], la1[kSets], lb0[kSets], lb1[kSets];  // CACHE = false: fragments that live for this pair only
        if (CACHE) {
            if (grp_a != ga) {  // warp-uniform
                ga = grp_a;
                load_frag(xq, grp_a, g, t, xa0, xa1);
            }
            if (have_b && grp_b != gb) {
                gb = grp_b;
                load_frag(xq, grp_b, g, t, xb0, xb1);
            }
        } else {
#pragma unroll
            for (int s = 0; s < kSets; s++) la0[s] = la1[s] = lb0[s] = lb1[s] = make_uint4(0, 0, 0, 0);
            load_frag(xq, grp_a, g, t, la0, la1);
            if (have_b) load_frag(xq, grp_b, g, t, lb0, lb1);
        }
        const uint4 (&fa0)[kSets] = CACHE ? xa0 : la0, (&fa1)[kSets] = CACHE ? xa1 : la1;
        const uint4 (&fb0)[kSets] = CACHE ? xb0 : lb0, (&fb1)[kSets] = CACHE ? xb1 : lb1;
        // Low and high nibbles go to separate accumulators: the low ones masked in place, the high ones masked in place
        // too (a byte 16 q, still a valid u8), so a word costs two logic operations and no shift.  The two chains are
        // independent; the fix-up adds them as 16 * low + high16, and the staged activation scale carries the 1/16.
        // B columns of a group: words (even positions, odd positions) of each 8-byte chunk: the low nibbles of a code
        // word are the even columns, the high nibbles the odd ones.
        constexpr unsigned ML = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
#pragma unroll
        for (int s = 0; s < kSets; s++) {
            int cal[4], cah[4], cbl[4], cbh[4];
            mma_u8s8_z(cal, a0.x & ML, a1.x & ML, a0.y & ML, a1.y & ML, fa0[s].x, fa0[s].z);
            mma_u8s8_z(cbl, b0.x & ML, b1.x & ML, b0.y & ML, b1.y & ML, fb0[s].x, fb0[s].z);
            mma_u8s8_z(cah, a0.x & MH, a1.x & MH, a0.y & MH, a1.y & MH, fa0[s].y, fa0[s].w);
            mma_u8s8_z(cbh, b0.x & MH, b1.x & MH, b0.y & MH, b1.y & MH, fb0[s].y, fb0[s].w);
            mma_u8s8(cal, a0.z & ML, a1.z & ML, a0.w & ML, a1.w & ML, fa1[s].x, fa1[s].z);
            mma_u8s8(cbl, b0.z & ML, b1.z & ML, b0.w & ML, b1.w & ML, fb1[s].x, fb1[s].z);
            mma_u8s8(cah, a0.z & MH, a1.z & MH, a0.w & MH, a1.w & MH, fa1[s].y, fa1[s].w);
            mma_u8s8(cbh, b0.z & MH, b1.z & MH, b0.w & MH, b1.w & MH, fb1[s].y, fb1[s].w);
            fix_up(cal, cah, tile_a, grp_a, meta, s, g, t);
            if (have_b) fix_up(cbl, cbh, tile_b, grp_b, meta, s, g, t);
        }
    }
    // One tile of 8-bit codes.  Tile layout (v2_repack8_kernel): four 512-byte planes [row g | row g + 8][column chunks
    // 0-1 | 2-3], 16 bytes per lane each = words (even columns of chunk j, odd columns of chunk j, even of j + 1, odd of
    // j + 1): the codes are u8 operands as they lie, the B fragments are the ones the 4-bit tiles use (the even / odd
    // split there comes from the nibble order).  The sums carry no factor 16, so the fix-up multiplies by it (exactly).
    __device__ __forceinline__ void single8(const unsigned char *tile, int grp, const uint32_t *xq, const float2 *meta, int lane) {
        const int g = lane >> 2, t = lane & 3;
        const uint4 a0 = *reinterpret_cast<const uint4 *>(tile + lane * 16);          // row g, chunks 0-1
        const uint4 a1 = *reinterpret_cast<const uint4 *>(tile + 512 + lane * 16);    // row g, chunks 2-3
        const uint4 c0 = *reinterpret_cast<const uint4 *>(tile + 1024 + lane * 16);   // row g + 8, chunks 0-1
        const uint4 c1 = *reinterpret_cast<const uint4 *>(tile + 1536 + lane * 16);   // row g + 8, chunks 2-3
        uint4 l0[kSets], l1[kSets];
        if (CACHE) {
            if (grp != ga) {
                ga = grp;
                load_frag(xq, grp, g, t, xa0, xa1);
            }
        } else {
#pragma unroll
            for (int s = 0; s < kSets; s++) l0[s] = l1[s] = make_uint4(0, 0, 0, 0);
            load_frag(xq, grp, g, t, l0, l1);
        }
        const uint4 (&f0)[kSets] = CACHE ? xa0 : l0, (&f1)[kSets] = CACHE ? xa1 : l1;
#pragma unroll
        for (int s = 0; s < kSets; s++) {
            int ce[4], co[4];
            mma_u8s8_z(ce, a0.x, c0.x, a0.z, c0.z, f0[s].x, f0[s].z);
            mma_u8s8_z(co, a0.y, c0.y, a0.w, c0.w, f0[s].y, f0[s].w);
            mma_u8s8(ce, a1.x, c1.x, a1.z, c1.z, f1[s].x, f1[s].z);
            mma_u8s8(co, a1.y, c1.y, a1.w, c1.w, f1[s].y, f1[s].w);
            const int b = 2 * s + (t >> 1);
            if (b < NB) {
                const float2 m = meta[(grp * NB + b) * 2 + (t & 1)];
                const __half2 *szp = reinterpret_cast<const __half2 *>(tile + TileGeom<8>::kCodeBytes);
                const float2 sz0 = __half22float2(szp[g]), sz1 = __half22float2(szp[g + 8]);
                const float f0v = fmaf((float)(ce[0] + co[0]), 4096.0f, (float)(ce[1] + co[1]) * 16.0f);
                const float f1v = fmaf((float)(ce[2] + co[2]), 4096.0f, (float)(ce[3] + co[3]) * 16.0f);
                acc0[s] = fmaf(sz0.x * m.x, fmaf(-sz0.y, m.y, f0v), acc0[s]);
                acc1[s] = fmaf(sz1.x * m.x, fmaf(-sz1.y, m.y, f1v), acc1[s]);
            }
        }
    }
    // Sums of rows g and g + 8 of batch row 2 s + t / 2, valid in both lanes of the pair afterwards.
    __device__ __forceinline__ void row_sums(int s, float &r0, float &r1) const {
        r0 = acc0[s] + __shfl_xor_sync(0xffffffffu, acc0[s], 1);
        r1 = acc1[s] + __shfl_xor_sync(0xffffffffu, acc1[s], 1);
    }
};

// One 8-element chunk of a group of 128 activations (the group's 16 chunks sit in 16 consecutive lanes: hl = lane & 15):
// round to 24-bit integers against the group's maximum, write the three byte planes in the fragment layout and, from
// the chunk's first lane, the two fix-up constants of (group, batch row).  v: the values to multiply the weights with.
template <int NB>
__device__ __forceinline__ void stage_chunk24(float (&v)[8], bool live, int grp, int b, int hl, uint32_t *xq, float2 *meta) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sx = amax > 0.0f ? amax * (1.0f / (float)kActTop) : 1.0f;
    const float inv = amax > 0.0f ? (float)kActTop / amax : 0.0f;
    // xi = hi * 65536 + mid * 256 + lo with signed digits: adding 0x808080 makes every digit a plain unsigned byte
    // (digit + 128, no carries between them), and flipping bit 7 of each byte turns that into the digit's two's complement.
    unsigned y[8];
    int lsum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int xi = __float2int_rn(v[i] * inv);
        xi = max(-kActTop, min(kActTop, xi));
        lsum += xi;
        y[i] = (unsigned)(xi + 0x808080) ^ 0x808080u;  // bytes: low, middle, high digit
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
    if (live) {
        const int t = hl >> 2, j = hl & 3;
        uint32_t *base = xq + ((((size_t)grp * 3 * NB + 3 * b) * 4 + t) * 4 + j) * 2;
#pragma unroll
        for (int c = 0; c < 3; c++) {  // staged plane c: 0 high, 1 middle, 2 low = byte 2 - c of y
            const unsigned sel = (unsigned)(2 - c) | ((unsigned)(6 - c) << 4);
            const unsigned e = __byte_perm(__byte_perm(y[0], y[2], sel), __byte_perm(y[4], y[6], sel), 0x5410);  // elements 0, 2, 4, 6
            const unsigned o = __byte_perm(__byte_perm(y[1], y[3], sel), __byte_perm(y[5], y[7], sel), 0x5410);  // elements 1, 3, 5, 7
            *reinterpret_cast<uint2 *>(base + 32 * c) = make_uint2(e, o);
        }
        if (hl == 0) {
            meta[(grp * NB + b) * 2] = make_float2(sx * 16.0f, (float)lsum * 0.0625f);
            meta[(grp * NB + b) * 2 + 1] = make_float2(sx * (1.0f / 4096.0f), 0.0f);
        }
    }
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kV2Consumers * 32) : "memory"); }


template <int S>
struct StageIterT {  // 32-bit and division-free in the loop: a 64-bit divide costs more than a tile
    int t, t_end, G, rb, grp;
    __device__ StageIterT(int t_begin, int t_end_, int G_) : t(t_begin), t_end(t_end_), G(G_), rb(t_begin / G_), grp(t_begin % G_) {}
    __device__ bool next(int &t0, int &n, int &rb0, int &grp0) {
        if (t >= t_end) return false;
        n = min(min(S, G - grp), t_end - t);
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
using StageIter = StageIterT<kStageTiles>;

}  // namespace im
