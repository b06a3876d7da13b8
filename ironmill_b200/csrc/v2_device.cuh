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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned i = 1;; i++) {
        __nanosleep(32);  // back off: a tight poll from many threads competes with the bulk copies for shared memory
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 0 && global_ns() - t0 > kWaitLimitNs) break;
    }
    atomicExch(err, 1);
    return false;
}
// One lane polls for the warp.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, int *err) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, err) ? 1 : 0;
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
