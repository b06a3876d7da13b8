// INT4 group-128 matvec, second generation: bulk-async staged, tensor-core dot products,
// stream-K work split.  Same arithmetic contract as matvec.cu (the (q - z) * s dequant of
// crates/ironmill-core/src/dequant.rs:129-139 applied to the decode projections
// crates/ironmill-inference/src/metal/shaders/quantized/affine_matvec.metal:16-111,
// affine_fused.metal:9-108, norm/superblock_fused_norm.metal:21-124).
//
// Layout (built once at load time): the matrix is cut into tiles of 16 rows x 128 columns
// (one quantization group): 16 x 64 bytes of nibbles = 1 KB, stored tile after tile in
// [row block][group] order, with the 16 (scale, zero) fp16 pairs of each tile in a parallel
// array.  A run of consecutive tiles is therefore one contiguous byte range, which one thread
// moves into shared memory with cp.async.bulk, completion counted on an mbarrier.  (A producer
// lane turns out one bulk copy per ~0.3 us whatever its size, so a stage is made large, 32 tiles = 34 KB.)
//
// Kernel: one persistent CTA per SM = 1 producer warp + 16 consumer warps around a ring of
// shared-memory stages (up to 32 tiles each), so the bytes in flight do not depend on how fast the
// consumers compute.  A consumer warp handles two tiles per stage: two 128-bit shared loads give
// each thread the 8 nibble words of its two rows, three logic operations per word split them
// into byte lanes, and four mma.sync m16n8k32 (u8 x s8 -> s32) multiply them with the
// activations, which were block-quantised once per CTA to 24-bit integers per 128-group (three
// signed byte planes in three B columns, the fourth column zero; two batch rows share one
// instruction, four a pass over the tile: TileMath, v2_device.cuh).
// Integer sums are exact inside a group; one float fix-up per tile applies
//   s * sx * (sum_k xi_k q_k - z * sum_k xi_k).
// Work is split stream-K fashion: every CTA gets the same number of tiles (+-1) out of the
// flattened [row block][group] list; a row block cut by a CTA boundary is completed by whichever
// of its CTAs arrives last (an atomic counter; nobody waits), summing the partials in CTA order
// so the result does not depend on arrival order.
#include "common.cuh"
#include "v2_device.cuh"

namespace im {

// Activation staging of batch row b (layout and rounding: stage_chunk24, v2_device.cuh).  Returns this thread's share
// of sum r^2 (residual + norm modes).
template <int MODE, int NB>
__device__ __forceinline__ float v2_stage_x(const V2Params &p, int b, uint32_t *xq, float2 *meta, int nthreads_warps) {
    const int K = p.K, lane = threadIdx.x & 31, hl = lane & 15, warp = threadIdx.x >> 5;
    float sq = 0.0f;
#pragma unroll 2
    for (int g0 = warp * 2; g0 < p.G; g0 += nthreads_warps * 2) {
        const int grp = g0 + (lane >> 4);
        const bool live = grp < p.G;
        const int k = (live ? grp : g0) * 128 + hl * 8;
        float v[8];
        {
            const uint4 raw = *reinterpret_cast<const uint4 *>(p.x + (size_t)b * K + k);
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(h[i]);
                v[2 * i] = f.x;
                v[2 * i + 1] = f.y;
            }
        }
        if (MODE & 2) {
            const uint4 rb = *reinterpret_cast<const uint4 *>(p.b + (size_t)b * K + k);
            const uint4 rg = *reinterpret_cast<const uint4 *>(p.gamma + k);
            const __half2 *hb = reinterpret_cast<const __half2 *>(&rb), *hg = reinterpret_cast<const __half2 *>(&rg);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 fb = __half22float2(hb[i]), fg = __half22float2(hg[i]);
                const float r0 = v[2 * i] + fb.x, r1 = v[2 * i + 1] + fb.y;
                if (live) sq += r0 * r0 + r1 * r1;
                v[2 * i] = r0 * fg.x;
                v[2 * i + 1] = r1 * fg.y;
            }
        }
        if (p.awq) {
            const uint4 ra = *reinterpret_cast<const uint4 *>(p.awq + k);
            const __half2 *ha = reinterpret_cast<const __half2 *>(&ra);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 fa = __half22float2(ha[i]);
                v[2 * i] = __fdiv_rn(v[2 * i], fa.x);
                v[2 * i + 1] = __fdiv_rn(v[2 * i + 1], fa.y);
            }
        }
        stage_chunk24<NB>(v, live, grp, b, hl, xq, meta);
    }
    return sq;
}

// MODE bit 0: gate+up+SiLU epilogue (tile rows 0-7 = gate rows, 8-15 = up rows of the same outputs);
// MODE bit 1: residual + RMSNorm prologue (x = (a + b) * gamma, outputs scaled by rms_inv).
//
// Stage schedule (the producer lane and every consumer warp walk the same list): the CTA owns the
// flattened tile range [t_begin, t_end); a stage is the next run of at most kStageTiles tiles that
// stays inside one row block.
template <int MODE, int NB, int BITS>
__global__ void __launch_bounds__(kV2Threads, 1) matvec_v2_kernel(const V2Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int G = p.G, nring = p.nring;
    using TG = TileGeom<BITS>;
    using Iter = StageIterT<TG::kStageTiles>;
    constexpr int kTileBytes = TG::kTileBytes;  // (shadows the 4-bit constants of the namespace on purpose)
    constexpr int stage_bytes = TG::kStageTiles * kTileBytes;
    unsigned char *ring = smem;                                                        // nring * stage_bytes
    uint32_t *xq = reinterpret_cast<uint32_t *>(ring + (size_t)nring * stage_bytes);   // G * 3NB * 32 words
    float2 *meta = reinterpret_cast<float2 *>(xq + (size_t)G * 3 * NB * 32);           // G * NB * 2
    float *red = reinterpret_cast<float *>(meta + (size_t)G * NB * 2);                 // nring * warps * 64 partial sums
    float *misc = red + (size_t)nring * kV2Consumers * 64;                             // 16 floats: rms_inv per batch row, reduction scratch
    uint64_t *full = reinterpret_cast<uint64_t *>(misc + 32);
    uint64_t *empty = full + nring;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int total = p.nblk * G;  // tiles (fits 32 bits: checked on the host)
    // Work split.  With enough row blocks each CTA takes whole row blocks: the kernel is HBM-bound, a CTA with
    // one block more than its neighbour simply keeps streaming while the others have left the bus, and no fix-up
    // is needed.  With few row blocks (short matrices) the split is by tiles, stream-K fashion (see flush()).
    const int t_begin = p.split_tiles ? (int)((long long)total * blockIdx.x / gridDim.x) : (int)((long long)p.nblk * blockIdx.x / gridDim.x) * G;
    const int t_end = p.split_tiles ? (int)((long long)total * (blockIdx.x + 1) / gridDim.x) : (int)((long long)p.nblk * (blockIdx.x + 1) / gridDim.x) * G;

    pdl_trigger();
    if (tid == 0) {
        for (int i = 0; i < nring; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kV2Consumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kV2Consumers) {
        // ------------------------------------------------ producer warp
        // Lane 0 streams the stages.  Before a ring slot is refilled the warp waits for the sixteen consumer warps
        // to release it; if the stage that lived there ended a row block, the consumers left their partial sums in
        // the slot's buffer and this otherwise idle warp adds them in warp order (so the result does not depend on
        // timing) and writes the outputs.  Consumers thus never wait for each other.
        // A row block cut by a CTA boundary (tile-granular split) is published as a partial instead; the last CTA
        // to arrive at its counter combines the partials in CTA order.
        const int bb = lane & 3, row = lane >> 2;  // lane owns entries e = lane (rows 0..7) and lane + 32 (rows 8..15)
        auto drain = [&](int slot, int rb) {
            const float *buf = red + slot * (kV2Consumers * 64);
            float v0 = 0.0f, v1 = 0.0f;
            if (bb < NB) {
#pragma unroll
                for (int w = 0; w < kV2Consumers; w++) {
                    v0 += buf[w * 64 + lane];
                    v1 += buf[w * 64 + lane + 32];
                }
            }
            const int b0 = rb * G, b1 = b0 + G;
            bool finalize = b0 >= t_begin && b1 <= t_end;
            if (!finalize) {
                const int pslot = (rb == t_begin / G) ? 0 : 1;
                float *mine = p.partial + ((size_t)blockIdx.x * 2 + pslot) * 64;
                mine[lane] = v0;
                mine[lane + 32] = v1;
                __threadfence();
                __syncwarp();
                const int c_first = (int)((((long long)b0 + 1) * gridDim.x + total - 1) / total) - 1;
                const int c_last = (int)(((long long)b1 * gridDim.x + total - 1) / total) - 1;
                int fin = 0;
                if (lane == 0) fin = atomicAdd(&p.counters[rb], 1) == c_last - c_first;
                finalize = __shfl_sync(0xffffffffu, fin, 0) != 0;
                if (finalize) {
                    __threadfence();
                    v0 = v1 = 0.0f;
                    for (int c = c_first; c <= c_last; c++) {
                        const int cb = (int)((long long)total * c / gridDim.x);
                        const float *theirs = p.partial + ((size_t)c * 2 + ((rb == cb / G) ? 0 : 1)) * 64;
                        v0 += __ldcg(theirs + lane);
                        v1 += __ldcg(theirs + lane + 32);
                    }
                    if (lane == 0) p.counters[rb] = 0;  // ready for the next launch
                }
            }
            if (finalize && bb < NB) {
                const float ri = (MODE & 2) ? misc[bb] : 1.0f;  // rms_inv, left by the consumers before their first release
                if (MODE & 1) {  // rows 0..7 gate, rows 8..15 up of the same eight outputs
                    const float gv = v0 * ri, uv = v1 * ri;
                    const int n = rb * 8 + row;
                    if (n < p.N) p.y[(size_t)bb * p.N + n] = __float2half_rn((gv / (1.0f + expf(-gv))) * uv);
                } else {
                    const int n = rb * 16 + row;
                    if (n < p.N) p.y[(size_t)bb * p.N + n] = __float2half_rn(v0 * ri);
                    if (n + 8 < p.N) p.y[(size_t)bb * p.N + n + 8] = __float2half_rn(v1 * ri);
                }
            }
        };
        Iter issue(t_begin, t_end, G), done(t_begin, t_end, G);
        int t0, n, rb0, grp0, dt0, dn, drb, dgrp;
        int slot = 0, phase = 0;  // slot of the stage being issued; phase = parity of the ring pass that last used it
        bool ok = true;
        int nstages = 0;
        for (; issue.next(t0, n, rb0, grp0); nstages++) {
            if (nstages >= nring) {  // reclaim: stage (nstages - nring) lived in this slot
                if (ok && !mbar_wait_warp(&empty[slot], phase ^ 1, p.err)) ok = false;
                done.next(dt0, dn, drb, dgrp);
                if (ok && (dgrp + dn == G || dt0 + dn == t_end)) drain(slot, drb);
            }
            if (lane == 0 && ok) {
                mbar_expect_tx(&full[slot], (uint32_t)(n * kTileBytes));
                bulk_g2s(ring + (size_t)slot * stage_bytes, p.tiles + (size_t)t0 * kTileBytes, (uint32_t)(n * kTileBytes), &full[slot]);
            }
            if (++slot == nring) {
                slot = 0;
                phase ^= 1;
            }
        }
        // the last min(nring, nstages) stages are still in the ring
        int left = nstages < nring ? nstages : nring;
        int dslot = nstages < nring ? 0 : slot, dphase = nstages < nring ? 0 : (phase ^ 1);
        for (; left > 0; left--) {
            if (ok && !mbar_wait_warp(&empty[dslot], dphase, p.err)) ok = false;
            done.next(dt0, dn, drb, dgrp);
            if (ok && (dgrp + dn == G || dt0 + dn == t_end)) drain(dslot, drb);
            if (++dslot == nring) {
                dslot = 0;
                dphase ^= 1;
            }
        }
        return;
    }

    // ---------------------------------------------------- consumers
    // The weights are constants, so the producer above streams them without waiting; the activations come
    // from the preceding kernel.  (The producer's output writes follow consumer releases, hence this wait.)
    pdl_wait();
    float sq_tot[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) {
        float sq = v2_stage_x<MODE, NB>(p, b, xq, meta, kV2Consumers);
        sq_tot[b] = 0.0f;
        if (MODE & 2) {
            sq = warp_sum(sq);
            if (lane == 0) misc[8 + warp] = sq;
            consumer_sync();
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < kV2Consumers; w++) t += misc[8 + w];
            sq_tot[b] = t;
            consumer_sync();
        }
    }
    consumer_sync();
    float rms_inv[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) rms_inv[b] = (MODE & 2) ? rsqrtf(sq_tot[b] / (float)p.K + p.eps) : 1.0f;
    if ((MODE & 2) && tid == 0) {
#pragma unroll
        for (int b = 0; b < NB; b++) misc[b] = rms_inv[b];  // visible to the producer warp through the slot-release barrier
    }
    if ((MODE & 2) && blockIdx.x == 0) {  // side outputs (must not alias a or b)
        for (int b = 0; b < NB; b++)
            for (int k = tid; k < p.K; k += kV2Consumers * 32) {
                const float r = __half2float(p.x[(size_t)b * p.K + k]) + __half2float(p.b[(size_t)b * p.K + k]);
                if (p.residual_out) p.residual_out[(size_t)b * p.K + k] = __float2half_rn(r);
                if (p.normed_out) p.normed_out[(size_t)b * p.K + k] = __float2half_rn(r * rms_inv[b] * __half2float(p.gamma[k]));
            }
    }

    const int g = lane >> 2, t = lane & 3;  // fragment coordinates: rows g and g+8, batch column pair t
    bool dead = false;
    TileMath<NB> tm;
    tm.reset();

    // A warp whose wait ran out stops computing but keeps every barrier of the schedule, so that
    // the other warps and the producer still run to the end; the host sees the error word.
    Iter it(t_begin, t_end, G);
    int t0, n, rb, grp0, slot = 0, phase = 0;
    while (it.next(t0, n, rb, grp0)) {
        if (!dead && !mbar_wait_warp(&full[slot], phase, p.err)) dead = true;
        const unsigned char *st = ring + (size_t)slot * stage_bytes;
        if (!dead && warp < n) {
            if (BITS == 4) {
                const int tb = warp + kV2Consumers;
                tm.pair(st + (size_t)warp * kTileBytes, grp0 + warp, st + (size_t)tb * kTileBytes, grp0 + tb, tb < n, xq, meta, lane);
            } else {
                tm.single8(st + (size_t)warp * kTileBytes, grp0 + warp, xq, meta, lane);
            }
        }
        if (grp0 + n == G || t0 + n == t_end) {  // last stage of this row block inside the CTA's range:
            float *buf = red + slot * (kV2Consumers * 64);  // hand the partial sums to the producer warp
#pragma unroll
            for (int cs = 0; cs < TileMath<NB>::kSets; cs++) {
                float r0, r1;
                tm.row_sums(cs, r0, r1);
                const int bb = 2 * cs + (t >> 1);
                if (!(t & 1) && bb < NB) {
                    buf[warp * 64 + g * 4 + bb] = r0;
                    buf[warp * 64 + (g + 8) * 4 + bb] = r1;
                }
            }
            tm.clear_sums();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
        if (++slot == nring) {
            slot = 0;
            phase ^= 1;
        }
    }
}

// ---- load-time repack -------------------------------------------------------
// Row-major codes [N][K/2] + interleaved (s, z) [N][G]  ->  tiles of 1088 bytes (1024 of nibbles: 16 rows x
// 64 bytes, then the 16 (scale, zero) pairs).  One thread per 16-byte chunk of nibbles.
// rows_per_blk = 16 (plain) or 8 (gate/up pair: tile rows 0-7 from matrix 0, 8-15 from matrix 1).
__global__ void v2_repack_kernel(const uint8_t *__restrict__ codes0, const __half2 *__restrict__ sz0, const uint8_t *__restrict__ codes1,
                                 const __half2 *__restrict__ sz1, int N, int K, int G, int nblk, int rows_per_blk,
                                 uint8_t *__restrict__ tiles) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // chunk index: ((rb*G + grp)*16 + r)*4 + c
    const size_t nchunks = (size_t)nblk * G * 64;
    if (i >= nchunks) return;
    const int c = i & 3, r = (i >> 2) & 15;
    const size_t tile = i >> 6;
    const int grp = (int)(tile % G), rb = (int)(tile / G);
    const bool second = rows_per_blk == 8 && r >= 8;
    const int row = rb * rows_per_blk + (rows_per_blk == 8 ? (r & 7) : r);
    const uint8_t *codes = second ? codes1 : codes0;
    const __half2 *sz = second ? sz1 : sz0;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < N) v = *reinterpret_cast<const uint4 *>(codes + (size_t)row * (K / 2) + grp * 64 + c * 16);
    uint8_t *dst = tiles + tile * kTileBytes;
    *reinterpret_cast<uint4 *>(dst + r * 64 + c * 16) = v;
    if (c == 0)
        reinterpret_cast<__half2 *>(dst + kTileCodeBytes)[r] =
            row < N ? sz[(size_t)row * G + grp] : __halves2half2(__float2half(0.0f), __float2half(0.0f));
}

int v2_repack(const uint8_t *codes0, const __half2 *sz0, const uint8_t *codes1, const __half2 *sz1, int N, int K, int G, int nblk,
              int rows_per_blk, uint8_t *tiles, cudaStream_t st) {
    const size_t nchunks = (size_t)nblk * G * 64;
    v2_repack_kernel<<<(unsigned)((nchunks + 255) / 256), 256, 0, st>>>(codes0, sz0, codes1, sz1, N, K, G, nblk, rows_per_blk, tiles);
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
}

// 8-bit codes: row-major [N][K] -> tiles of 2112 bytes in the plane order TileMath::single8 reads.  One thread per 16-byte
// chunk: chunk i of a tile = plane (i >> 5) = 2 * (row half) + (column part), lane i & 31 = (g, t); its source is the 16
// consecutive codes of row g + 8 * half at columns 32 t + 16 * part, split into (even, odd) bytes per 8 columns.
__global__ void v2_repack8_kernel(const uint8_t *__restrict__ codes, const __half2 *__restrict__ sz, int N, int K, int G, int nblk,
                                  uint8_t *__restrict__ tiles) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nchunks = (size_t)nblk * G * 128;
    if (i >= nchunks) return;
    const int lane = i & 31, part = (i >> 5) & 1, half = (i >> 6) & 1;
    const size_t tile = i >> 7;
    const int grp = (int)(tile % G), rb = (int)(tile / G);
    const int g = lane >> 2, t = lane & 3, r = g + 8 * half, row = rb * 16 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < N) v = *reinterpret_cast<const uint4 *>(codes + (size_t)row * K + grp * 128 + 32 * t + 16 * part);
    uint8_t *dst = tiles + tile * TileGeom<8>::kTileBytes;
    *reinterpret_cast<uint4 *>(dst + (2 * half + part) * 512 + lane * 16) =
        make_uint4(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531), __byte_perm(v.z, v.w, 0x6420), __byte_perm(v.z, v.w, 0x7531));
    if (part == 0 && t == 0)
        reinterpret_cast<__half2 *>(dst + TileGeom<8>::kCodeBytes)[r] =
            row < N ? sz[(size_t)row * G + grp] : __halves2half2(__float2half(0.0f), __float2half(0.0f));
}

int v2_repack8(const uint8_t *codes, const __half2 *sz, int N, int K, int G, int nblk, uint8_t *tiles, cudaStream_t st) {
    const size_t nchunks = (size_t)nblk * G * 128;
    v2_repack8_kernel<<<(unsigned)((nchunks + 255) / 256), 256, 0, st>>>(codes, sz, N, K, G, nblk, tiles);
    IM_CUDA_CHECK(cudaGetLastError());
    return IM_OK;
}

template <int MODE, int NB, int BITS = 4>
static int v2_launch(V2Params p, const Device *dev, cudaStream_t st) {
    const size_t stage_bytes = (size_t)TileGeom<BITS>::kStageTiles * TileGeom<BITS>::kTileBytes;
    const size_t red_buf = (size_t)kV2Consumers * 64 * 4;  // one partial-sum buffer per ring slot
    const size_t fixed = (size_t)p.G * 3 * NB * 32 * 4 + (size_t)p.G * NB * 16 + 32 * 4 + 64;
    const size_t per_slot = stage_bytes + 16 + red_buf;
    const size_t budget = dev->smem_optin > 8192 ? dev->smem_optin - 2048 : 0;
    if (fixed + 3 * per_slot > budget) return IM_ERR_BOUNDS;  // caller falls back to the first-generation kernel
    int nring = (int)((budget - fixed) / per_slot);
    if (nring > 8) nring = 8;
    p.nring = nring;
    const size_t smem = fixed + (size_t)nring * per_slot;
    auto kern = matvec_v2_kernel<MODE, NB, BITS>;
    static DeviceOnce once;  // per instantiation
    if (once.first(dev->ordinal)) IM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev->smem_optin));
    const long long total = (long long)p.nblk * p.G;
    if (total > 0x7fffffffLL) return IM_ERR_BOUNDS;
    int grid = dev->sm_count;
    p.split_tiles = p.nblk < grid ? 1 : 0;
    if (grid > total) grid = (int)total;
    IM_CUDA_CHECK(launch_k(kern, dim3(grid), dim3(kV2Threads), smem, st, p));
    return IM_OK;
}

// mode: bit 0 gate+up epilogue (paired tiles), bit 1 residual+norm prologue.  IM_ERR_BOUNDS if the shape does not fit.
int v2_run(int mode, int nb, const V2Params &p, const Device *dev, cudaStream_t st, int bits) {
    if (bits == 8) {  // 8-bit codes: the plain projection only (the reference has no fused 8-bit kernels)
        if (mode != 0) return IM_ERR_BOUNDS;
        if (nb == 1) return v2_launch<0, 1, 8>(p, dev, st);
        if (nb == 2) return v2_launch<0, 2, 8>(p, dev, st);
        if (nb == 4) return v2_launch<0, 4, 8>(p, dev, st);
        return fail(IM_ERR_INVALID, "unsupported v2 matvec batch %d", nb);
    }
#define V2_CASE(M, B) \
    if (mode == M && nb == B) return v2_launch<M, B>(p, dev, st);
    V2_CASE(0, 1) V2_CASE(0, 2) V2_CASE(0, 4) V2_CASE(1, 1) V2_CASE(1, 2) V2_CASE(1, 4) V2_CASE(2, 1) V2_CASE(2, 2) V2_CASE(2, 4) V2_CASE(3, 1) V2_CASE(3, 2) V2_CASE(3, 4)
#undef V2_CASE
    return fail(IM_ERR_INVALID, "unsupported v2 matvec mode %d / batch %d", mode, nb);
}

}  // namespace im
