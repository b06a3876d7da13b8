// INT4 group-128 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for the dense-contraction cases of the
// hot path: prefill chunks and decode batches of 16 tokens and more.
//   crates/ironmill-inference/src/metal/shaders/quantized/affine_matmul.metal:10-152 (superblock_matmul_int4):
//   C[m, n] = sum_k f16(A[m, k] / awq[k]) * f16((q[n, k] - z) * s), f32 accumulation, fp16 result.
//
// Shape of the computation: D[128 weight rows x TN tokens] (f32, in tensor memory) += W[128 x 16] * X[TN x 16]^T, issued
// by one thread with tcgen05.mma (kind::f16, UMMA M = 128, N = TN, K = 16), eight per stage of one quantisation
// group (128 columns).  Both operands sit in shared memory, K-major with the 128-byte swizzle:
//   * A: the weights.  Eight warps (thread = row and half of the group) read the packed 4-bit codes, 32 bytes per
//     thread and stage, and the row's (scale, zero), dequantise in packed fp16 arithmetic - (q - z) * s with one
//     rounding, the reference's f16((q - z) s) - and store fp16 straight into the swizzled operand layout: the
//     dequantisation is fused into the operand load, HBM carries 4 bits per weight.  The codes of the next stage
//     are requested before the current one is converted;
//   * B: the activations, already divided by the AWQ scales and rounded to fp16 (act_scale_kernel), brought in by
//     the copy engine: one thread issues two cp.async.bulk.tensor copies per stage (boxes of 64 columns x TN token
//     rows of a 2-D tensor map with the 128-byte swizzle; rows past the last token come back as zeros), completion
//     counted in bytes on the stage's full barrier.  The map covers this GPU's own buffer; no multicast.
// A ring of stages decouples the producers from the tensor core: full barriers count the eight weight warps and the
// announcement of the activation bytes, tcgen05.commit releases a stage when its eight MMAs have read it.  After the last group warps 0-3 read their 32
// TMEM lanes each (tcgen05.ld 32x32b), convert and write fp16 outputs.  Every wait is bounded; a wait that runs
// out sets the device error word, the kernel still frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "v2_device.cuh"

namespace im {

namespace {

constexpr int kGM = 128;       // weight rows per CTA = UMMA M
constexpr int kGK = 128;       // columns per stage = one quantisation group = two 64-column swizzle atoms
constexpr int kGAhead = 4;      // stages of packed codes a weight thread keeps in flight in registers (eight measured 5-15 % slower)
constexpr int kGWarpsA = 16, kGWarpsB = 1;      // warps 0-15: weights (0-3 also the epilogue), 16: activation copies, 17: tensor memory + MMA issue
constexpr int kGThreads = (kGWarpsA + kGWarpsB + 1) * 32;
constexpr int kGMmaWarp = kGWarpsA + kGWarpsB;

__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    // shared-memory matrix descriptor, K-major, 128-byte swizzle: start address >> 4 in bits 0-13, leading byte
    // offset (unused for swizzled K-major) = 1 in bits 16-29, stride byte offset = 1024 B (8 rows of 128 B) >> 4 in
    // bits 32-45, descriptor version 1 in bits 46-47, layout type 2 (SWIZZLE_128B) in bits 61-63
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One tile of the activation matrix: box {64 columns, TN rows} of a 2-D tensor map (fp16, 128-byte swizzle), landing in
// the K-major operand layout the MMA descriptors name; rows past the last token are filled with zeros.  Completion is
// counted in bytes on the stage's full barrier.  x is a multiple of 64 columns (128 bytes): the 16-byte rule holds.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

struct GemmParams {
    const uint8_t *codes;  // [N, K/2] row-major 4-bit codes, low nibble first
    const __half2 *sz;     // [N, G] (scale, zero)
    const __half *xs;      // [M, K] activations, already divided by the AWQ scales
    __half *y;             // [M, N]
    int N, K, G, M;
    int *err;
    // K split (few tokens, few row tiles): CTA z covers groups [z * gps, min(G, (z + 1) * gps)) and leaves its f32 sums in
    // partial[z][m][n]; gemm_splitk_reduce_kernel adds the slices in z order and rounds once.  partial == nullptr: one
    // CTA per tile covers every group and writes fp16 itself.
    float *partial;
    int gps;
};

// 8 nibbles of a word -> 8 fp16 values (q - z) * s in memory order.  c = 1024 + z, exact for integer z in
// [-1024, 1023]: 0x6400 | q is the fp16 number 1024 + q, the subtraction is exact, the product is rounded once.
__device__ __forceinline__ uint4 dequant8_fast(uint32_t w, __half2 c, __half2 s) {
    constexpr uint32_t M = 0x000F000Fu, E = 0x64006400u;
    uint32_t h04 = (w & M) | E, h15 = ((w >> 4) & M) | E, h26 = ((w >> 8) & M) | E, h37 = ((w >> 12) & M) | E;
    __half2 v04 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h04), c), s);
    __half2 v15 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h15), c), s);
    __half2 v26 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h26), c), s);
    __half2 v37 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h37), c), s);
    const uint32_t a = *reinterpret_cast<uint32_t *>(&v04), b = *reinterpret_cast<uint32_t *>(&v15);
    const uint32_t cc = *reinterpret_cast<uint32_t *>(&v26), d = *reinterpret_cast<uint32_t *>(&v37);
    return make_uint4(__byte_perm(a, b, 0x5410), __byte_perm(cc, d, 0x5410), __byte_perm(a, b, 0x7632), __byte_perm(cc, d, 0x7632));
}
// 8-bit codes: the 8 bytes of two words -> 8 fp16 values (q - z) * s in memory order.  0x6400 | q is 1024 + q for q < 1024.
__device__ __forceinline__ uint4 dequant8b_fast(uint32_t w0, uint32_t w1, __half2 c, __half2 s) {
    uint32_t h[4] = {__byte_perm(w0, 0x64u, 0x4140), __byte_perm(w0, 0x64u, 0x4342), __byte_perm(w1, 0x64u, 0x4140), __byte_perm(w1, 0x64u, 0x4342)};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h[i]), c), s);
        o[i] = *reinterpret_cast<const uint32_t *>(&v);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
__device__ __forceinline__ uint4 dequant8b_slow(uint32_t w0, uint32_t w1, float z, float s) {
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t w = i < 2 ? w0 : w1;
        const float lo = ((float)((w >> (16 * (i & 1))) & 255u) - z) * s, hi = ((float)((w >> (16 * (i & 1) + 8)) & 255u) - z) * s;
        o[i] = (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
__device__ __forceinline__ uint4 dequant8_slow(uint32_t w, float z, float s) {  // any zero point: f32, one rounding
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float lo = ((float)((w >> (8 * i)) & 15u) - z) * s, hi = ((float)((w >> (8 * i + 4)) & 15u) - z) * s;
        o[i] = (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// ring depth by token tile: 96 KB per stage at TN = 256 leaves room for two, 64 KB at TN = 128 for three (deeper rings
// measured no faster: the weight warps, not the pipeline depth, set the pace)
// (also for the small token tiles: five stages with four activation copies in flight at 32 tokens, four with three at
// 64, measured 20-60 % slower than three stages with two in flight on 16-64 tokens)
// Two 256-token tiles per dequantised weight stage (512 tokens per CTA, all of tensor memory) were built and measured at
// 2048 tokens: 2.5 us per pair of products = the 136 KB of operands a CTA then pulls per group at ~54 GB/s per SM, i.e.
// the L2 -> SM bandwidth bounds the activation supply, not the weight warps: +5-11 % where the CTAs formed one wave
// (o, down), -17 % where they did not (qkv); not kept.  Halving the activation bytes per product needs CTA pairs
// (cta_group::2) that share one activation tile.
template <int TN>
constexpr int gemm_stages() { return TN >= 256 ? 2 : 3; }

// The weight warps' work for one CTA: dequantise the groups [g_begin, g_begin + G) of rows n0 .. n0 + 127 into the A ring
// (STAGES slots of 32 KB), one stage per group; full barriers are arrived at once per warp and stage, empty barriers
// are waited on before a slot is reused.
template <int BITS, int STAGES>
__device__ __forceinline__ void gemm_weight_warps(const GemmParams &p, unsigned char *As, uint64_t *full, uint64_t *empty, int g_begin, int G, int n0,
                                                  bool &ok) {
    constexpr int kGStages = STAGES;
    constexpr int kABytes = kGM * kGK * 2;
    constexpr int kCodeVec = BITS == 4 ? 1 : 2;      // 16-byte vectors of codes per thread and stage (32 columns)
    constexpr int kAheadA = BITS == 4 ? kGAhead : 2;  // stages of codes in flight in registers (16 registers either way)
    const int tid = threadIdx.x, lane = tid & 31;
    // ---------------------------------------------------------------- weights: dequantise into operand A
    // thread = (row r, quarter q of the group): 32 columns = 16 (4-bit) or 32 (8-bit) bytes of codes per stage, four
    // 16-byte chunks of one swizzle atom.  The codes of the next stages are requested before this stage is converted,
    // so the memory latency is paid once.  Sixteen such warps: four per scheduler to cover each other's dependent
    // chains (eight measured 43 % issue utilisation).
    const int r = tid & 127, q = tid >> 7, n = n0 + r;
    const bool live = n < p.N;
    const uint8_t *crow = p.codes + (size_t)(live ? n : 0) * ((size_t)p.K * BITS / 8) + (size_t)g_begin * (16 * BITS) + q * (4 * BITS);
    const __half2 *szrow = p.sz + (size_t)(live ? n : 0) * p.G + g_begin;
    const uint32_t row_off = (uint32_t)((q >> 1) * (kGM * 128) + (r >> 3) * 1024 + (r & 7) * 128);
    const int c0 = 4 * (q & 1);  // first 16-byte chunk of this thread inside the atom's 128-byte row
    // register ring of the next kAheadA stages' codes: 16 (4-bit) or 32 (8-bit) bytes per stage in flight per thread,
    // enough to cover the memory latency at one stage per ~0.3 us
    uint4 wb[kAheadA][kCodeVec];
    __half2 szb[kAheadA];
#pragma unroll
    for (int u = 0; u < kAheadA; u++) {
#pragma unroll
        for (int v = 0; v < kCodeVec; v++) wb[u][v] = make_uint4(0, 0, 0, 0);
        szb[u] = __floats2half2_rn(0.0f, 0.0f);
        if (live && u < G) {
            const uint4 *src = reinterpret_cast<const uint4 *>(crow + (size_t)u * (16 * BITS));
#pragma unroll
            for (int v = 0; v < kCodeVec; v++) wb[u][v] = ldg_stream_v4(src + v);
            szb[u] = szrow[u];
        }
    }
    for (int kt0 = 0; kt0 < G; kt0 += kAheadA) {
#pragma unroll
        for (int u = 0; u < kAheadA; u++) {
            const int kt = kt0 + u;
            if (kt < G) {  // warp-uniform
                const int s = kt % kGStages, use = kt / kGStages;
                uint4 cw[kCodeVec];
#pragma unroll
                for (int v = 0; v < kCodeVec; v++) cw[v] = wb[u][v];
                const __half2 szc = szb[u];
                if (live && kt + kAheadA < G) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(crow + (size_t)(kt + kAheadA) * (16 * BITS));
#pragma unroll
                    for (int v = 0; v < kCodeVec; v++) wb[u][v] = ldg_stream_v4(src + v);
                    szb[u] = szrow[kt + kAheadA];
                }
                // convert into registers first: only the eight stores wait for the slot to be free
                const float zf = __high2float(szc), sf = __low2float(szc);
                const bool fast = zf == rintf(zf) && zf >= -1024.0f && zf <= 1023.0f;
                uint4 v0, v1, v2, v3;
                // Two real branches (not a select): the f32 path costs three times the packed one and almost no group
                // needs it.  Rows past N carry zero codes and a zero scale, which dequantise to zero.
                if (__builtin_expect(fast, 1)) {
                    const __half2 c2 = __float2half2_rn(1024.0f + zf), s2 = __half2half2(__low2half(szc));
                    if (BITS == 4) {
                        v0 = dequant8_fast(cw[0].x, c2, s2); v1 = dequant8_fast(cw[0].y, c2, s2); v2 = dequant8_fast(cw[0].z, c2, s2); v3 = dequant8_fast(cw[0].w, c2, s2);
                    } else {
                        v0 = dequant8b_fast(cw[0].x, cw[0].y, c2, s2); v1 = dequant8b_fast(cw[0].z, cw[0].w, c2, s2);
                        v2 = dequant8b_fast(cw[kCodeVec - 1].x, cw[kCodeVec - 1].y, c2, s2); v3 = dequant8b_fast(cw[kCodeVec - 1].z, cw[kCodeVec - 1].w, c2, s2);
                    }
                } else if (BITS == 4) {
                    v0 = dequant8_slow(cw[0].x, zf, sf); v1 = dequant8_slow(cw[0].y, zf, sf); v2 = dequant8_slow(cw[0].z, zf, sf); v3 = dequant8_slow(cw[0].w, zf, sf);
                } else {
                    v0 = dequant8b_slow(cw[0].x, cw[0].y, zf, sf); v1 = dequant8b_slow(cw[0].z, cw[0].w, zf, sf);
                    v2 = dequant8b_slow(cw[kCodeVec - 1].x, cw[kCodeVec - 1].y, zf, sf); v3 = dequant8b_slow(cw[kCodeVec - 1].z, cw[kCodeVec - 1].w, zf, sf);
                }
                if (ok && use > 0 && !mbar_wait_warp(&empty[s], (use - 1) & 1, p.err)) ok = false;
                unsigned char *dst = As + (size_t)s * kABytes + row_off;
                const int x = r & 7;  // chunk c = columns 8c .. 8c + 7 of the atom's 64, stored at chunk c ^ (row & 7)
                *reinterpret_cast<uint4 *>(dst + (((c0 + 0) ^ x) << 4)) = v0;
                *reinterpret_cast<uint4 *>(dst + (((c0 + 1) ^ x) << 4)) = v1;
                *reinterpret_cast<uint4 *>(dst + (((c0 + 2) ^ x) << 4)) = v2;
                *reinterpret_cast<uint4 *>(dst + (((c0 + 3) ^ x) << 4)) = v3;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
            }
        }
    }
}

template <int TN, int BITS>
__global__ void __launch_bounds__(kGThreads, 1) gemm_int4_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_b) {
    constexpr int kGStages = gemm_stages<TN>();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of every operand buffer: the swizzle is a function of the address bits
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int kABytes = kGM * kGK * 2, kBBytes = TN * kGK * 2;
    unsigned char *As = smem, *Bs = smem + kGStages * kABytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(Bs + kGStages * kBBytes);
    uint64_t *empty = full + kGStages;
    uint64_t *accum = empty + kGStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * kGM, m0 = blockIdx.y * TN;
    pdl_trigger();
    if (tid == 0) {
        for (int i = 0; i < kGStages; i++) {
            mbar_init(&full[i], kGWarpsA + 1);  // the weight warps + the thread that announces the activation bytes
            mbar_init(&empty[i], 1);
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kGMmaWarp) {  // TN f32 columns of tensor memory for the accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TN < 32 ? 32 : TN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    pdl_wait();

    const int g_begin = blockIdx.z * p.gps;
    const int G = min(p.G, g_begin + p.gps) - g_begin;  // this CTA's groups (stages), >= 1 by construction of the grid
    bool ok = true;
    if (warp < kGWarpsA) {
        gemm_weight_warps<BITS, kGStages>(p, As, full, empty, g_begin, G, n0, ok);
    } else if (warp == kGWarpsA) {
        // ---------------------------------------------------------------- activations: TMA into operand B
        // One thread per stage: wait for the slot, announce the bytes on the stage's full barrier and issue the two
        // tensor copies (columns 0-63 and 64-127 of the group, TN token rows each; a tensor map over this GPU's own
        // activation buffer, no multicast).  The copy engine does the swizzle and the zero fill of rows past M.
        for (int it = 0; it < G; it++) {
            const int s = it % kGStages, use = it / kGStages;
            if (ok && use > 0 && !mbar_wait_warp(&empty[s], (use - 1) & 1, p.err)) ok = false;
            if (lane == 0 && ok) {
                unsigned char *dst = Bs + (size_t)s * kBBytes;
                const int x = (g_begin + it) * kGK;
                mbar_expect_tx(&full[s], (uint32_t)kBBytes);
                tma_load_2d(dst, &tmap_b, x, m0, &full[s]);
                tma_load_2d(dst + TN * 128, &tmap_b, x + 64, m0, &full[s]);
            }
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------------------- one thread issues the MMAs
        // instruction descriptor: f32 accumulator (bit 4), fp16 A and B (formats 0), both K-major, N >> 3 in bits
        // 17-22, M >> 4 in bits 24-28
        constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(kGM >> 4) << 24);
        for (int kt = 0; kt < G; kt++) {
            const int s = kt % kGStages, use = kt / kGStages;
            if (ok && !mbar_wait_warp(&full[s], use & 1, p.err)) ok = false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0 && ok) {
                const uint32_t a0 = smem_u32(As + (size_t)s * kABytes), b0 = smem_u32(Bs + (size_t)s * kBBytes);
#pragma unroll
                for (int j = 0; j < 8; j++) {  // K = 16 per instruction: 32 bytes along the swizzled row, second atom after four
                    const uint64_t ad = umma_desc_sw128(a0 + (j >> 2) * (kGM * 128) + (j & 3) * 32);
                    const uint64_t bd = umma_desc_sw128(b0 + (j >> 2) * (TN * 128) + (j & 3) * 32);
                    umma_f16(tmem_d, ad, bd, idesc, (kt > 0 || j > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);              // the stage is free once these MMAs have read it
                if (kt == G - 1) umma_commit(accum);  // ... and the accumulator is complete after the last one
            }
            __syncwarp();
        }
    }

    // -------------------------------------------------------------------- epilogue: TMEM -> fp16 outputs
    if (warp < 4) {
        if (ok && !mbar_wait_warp(accum, 0, p.err)) ok = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int n = n0 + tid;  // this thread's TMEM lane = weight row
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < TN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
                if (n < p.N) {
                    if (p.partial) {
                        float *dst = p.partial + (size_t)blockIdx.z * p.M * p.N + n;
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            const int m = m0 + c0 + i;
                            if (m < p.M) dst[(size_t)m * p.N] = __uint_as_float(r[i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            const int m = m0 + c0 + i;
                            if (m < p.M) p.y[(size_t)m * p.N + n] = __float2half_rn(__uint_as_float(r[i]));
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kGMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TN < 32 ? 32 : TN) : "memory");
    }
}

// xs[m, k] = f16(x[m, k] / awq[k]) (or a copy when there are no activation scales)
__global__ void act_scale_kernel(const __half *__restrict__ x, const __half *__restrict__ awq, __half *__restrict__ xs, size_t n, int K) {
    pdl_trigger();
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    uint4 v = *reinterpret_cast<const uint4 *>(x + i);
    if (awq) {
        const uint4 a = *reinterpret_cast<const uint4 *>(awq + (i % (size_t)K));
        __half2 *hv = reinterpret_cast<__half2 *>(&v);
        const __half2 *ha = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 fx = __half22float2(hv[j]), fa = __half22float2(ha[j]);
            hv[j] = __floats2half2_rn(fx.x / fa.x, fx.y / fa.y);
        }
    }
    *reinterpret_cast<uint4 *>(xs + i) = v;
}

// y[i] = f16(partial[0][i] + partial[1][i] + ...), slices added in order: one rounding, as the unsplit kernel's epilogue
__global__ void gemm_splitk_reduce_kernel(const float *__restrict__ partial, __half *__restrict__ y, size_t n, int splits) {
    pdl_trigger();
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 a = *reinterpret_cast<const float4 *>(partial + i);
    for (int z = 1; z < splits; z++) {
        const float4 b = *reinterpret_cast<const float4 *>(partial + (size_t)z * n + i);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    const __half2 lo = __floats2half2_rn(a.x, a.y), hi = __floats2half2_rn(a.z, a.w);
    *reinterpret_cast<uint2 *>(y + i) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda).
typedef CUresult (*TmapEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TmapEncodeFn tmap_encode_fn() {
    static TmapEncodeFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<TmapEncodeFn>(f);
    }();
    return fn;
}

// activations [M, K] fp16 row-major as a 2-D tensor: inner dimension K, boxes of 64 columns x `rows` rows, 128-byte swizzle
static int make_act_tmap(const GemmParams &p, int rows, CUtensorMap *tmap) {
    TmapEncodeFn enc = tmap_encode_fn();
    if (!enc) return fail(IM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t gdim[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
    const cuuint64_t gstride[1] = {(cuuint64_t)p.K * sizeof(__half)};
    const cuuint32_t box[2] = {64u, (cuuint32_t)rows};
    const cuuint32_t estride[2] = {1u, 1u};
    const CUresult cr = enc(tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(p.xs), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(IM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for activations [%d, %d]", (int)cr, p.M, p.K);
    return IM_OK;
}

template <int TN, int BITS>
int gemm_launch(const GemmParams &p, const Device *dev, cudaStream_t st) {
    constexpr int kGStages = gemm_stages<TN>();
    const size_t smem = 1024 + (size_t)kGStages * (kGM * kGK * 2 + TN * kGK * 2) + (2 * kGStages + 1) * 8 + 16;
    if (smem > dev->smem_optin) return IM_ERR_BOUNDS;
    auto kern = gemm_int4_tc_kernel<TN, BITS>;
    static DeviceOnce once;  // per instantiation
    if (once.first(dev->ordinal)) IM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    alignas(64) CUtensorMap tmap;
    if (const int trc = make_act_tmap(p, TN, &tmap); trc != IM_OK) return trc;
    const int splits = (p.G + p.gps - 1) / p.gps;
    dim3 grid((p.N + kGM - 1) / kGM, (p.M + TN - 1) / TN, splits);
    IM_CUDA_CHECK(launch_k(kern, grid, dim3(kGThreads), smem, st, p, tmap));
    if (p.partial) {
        const size_t n = (size_t)p.M * p.N;  // N is a multiple of 4 here (checked by the caller)
        IM_CUDA_CHECK(launch_k(gemm_splitk_reduce_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, st, (const float *)p.partial, p.y, n, splits));
    }
    return IM_OK;
}

}  // namespace

// Y[M, N] = f16(X / awq) * dequant(W)^T for M tokens.  xs_scratch: M * K halves.  IM_ERR_BOUNDS when the weight is not
// INT4 group-128 with K a multiple of 128 (the caller falls back to the matvec kernels).
int gemm_affine_tc(const AffineWeight *w, const __half *x, __half *y, int M, __half *xs_scratch, cudaStream_t st) {
    if ((w->bits != 4 && w->bits != 8) || w->group_size != 128 || w->K % 128 != 0 || M < 1) return IM_ERR_BOUNDS;
    const size_t n = (size_t)M * w->K;
    IM_CUDA_CHECK(launch_k(act_scale_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, x, (const __half *)w->awq, xs_scratch, n, w->K));
    GemmParams p{w->codes, w->sz, xs_scratch, y, w->N, w->K, w->G, M, w->dev->err_flag, nullptr, w->G};
    // Few tokens and few row tiles (decode batches of 16-64 against 4096-6144 rows: 32-48 CTAs of 32-112 sequential
    // stages): split K so that the grid covers the GPU.  At least four groups per slice; the slices' f32 sums go through
    // the device handle's scratch (one GEMM in flight per handle, like the tiled matvec).
    if (M <= 64 && w->N % 4 == 0 && w->dev->gemm_partial) {
        const int tiles = (w->N + kGM - 1) / kGM;
        int splits = std::min(w->dev->sm_count / tiles, w->G / 4);
        while (splits > 1 && (size_t)splits * M * w->N * sizeof(float) > kGemmPartialBytes) splits--;
        if (splits > 1) {
            p.gps = (w->G + splits - 1) / splits;
            p.partial = w->dev->gemm_partial;
        }
    }
    // a 256-token tile shares every dequantised weight tile between twice as many tokens, but halves the CTA count:
    // worth it only once the grid still covers the GPU
    const long long ctas256 = (long long)((w->N + kGM - 1) / kGM) * ((M + 255) / 256);
    if (w->bits == 8) {  // superblock_matmul_int8 (affine_matmul.metal:155-290): the same kernel, byte codes
        if (M > 128 && ctas256 >= w->dev->sm_count) return gemm_launch<256, 8>(p, w->dev, st);
        if (M > 64) return gemm_launch<128, 8>(p, w->dev, st);
        if (M > 32) return gemm_launch<64, 8>(p, w->dev, st);
        return gemm_launch<32, 8>(p, w->dev, st);
    }
    if (M > 128 && ctas256 >= w->dev->sm_count) return gemm_launch<256, 4>(p, w->dev, st);
    if (M > 64) return gemm_launch<128, 4>(p, w->dev, st);
    if (M > 32) return gemm_launch<64, 4>(p, w->dev, st);
    return gemm_launch<32, 4>(p, w->dev, st);
}

}  // namespace im
