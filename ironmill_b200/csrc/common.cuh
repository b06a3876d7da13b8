// Shared helpers for the sm_100a decode kernels and their C ABI.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>
#include <string>

#include "../../include/ironmill_cuda.h"

#define IM_EXPORT extern "C" __attribute__((visibility("default")))

namespace im {

// Thread-local error text behind im_cuda_last_error().
std::string &last_error();
int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

#define IM_CUDA_CHECK(expr)                                                                   \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            return im::fail(_e == cudaErrorMemoryAllocation ? IM_ERR_ALLOC : IM_ERR_CUDA,     \
                            "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, \
                            __LINE__);                                                        \
    } while (0)

#define IM_REQUIRE(cond, ...)                               \
    do {                                                    \
        if (!(cond)) return im::fail(IM_ERR_INVALID, __VA_ARGS__); \
    } while (0)

// Wrap an entry point body so that no C++ exception crosses the C boundary.
#define IM_GUARD_BEGIN try {
#define IM_GUARD_END                                                        \
    }                                                                       \
    catch (const std::bad_alloc &) { return im::fail(IM_ERR_ALLOC, "host allocation failed"); } \
    catch (const std::exception &e) { return im::fail(IM_ERR_CUDA, "exception: %s", e.what()); } \
    catch (...) { return im::fail(IM_ERR_CUDA, "unknown exception"); }

struct Device {
    int ordinal = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    cudaDeviceProp prop{};
    size_t allocated = 0;  // bytes handed out through this handle
    // stream-K scratch of the tiled matvec: partial sums of row blocks cut by a CTA boundary and the
    // arrival counters of those blocks.  One matvec in flight per device handle at a time.
    float *sk_partial = nullptr;
    int *sk_counters = nullptr;
    int *err_flag = nullptr;  // set by a kernel whose bounded wait ran out
    // f32 slices of a K-split tensor-core GEMM (gemm_tc.cu; few tokens against few row tiles).  One GEMM in flight per
    // device handle at a time.
    float *gemm_partial = nullptr;
};
constexpr size_t kGemmPartialBytes = (size_t)8 << 20;
constexpr int kSkMaxBlocks = 1 << 17;  // row blocks the counters cover (2M rows)

// cudaFuncSetAttribute applies to the current device: remember per device ordinal (not per thread) whether a
// kernel's attribute has been set.  Usage: static DeviceOnce once; if (once.first(dev->ordinal)) { set attributes }.
struct DeviceOnce {
    std::atomic<bool> done[64];
    DeviceOnce() {
        for (auto &d : done) d.store(false);
    }
    bool first(int ordinal) {
        if (ordinal < 0 || ordinal >= 64) return true;  // outside the table: set every time
        return !done[ordinal].exchange(true);
    }
};

// Allocation bookkeeping shared by buffers, weights and models.
int dev_malloc(Device *dev, void **ptr, size_t bytes);
void dev_free(Device *dev, void *ptr, size_t bytes);

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// GPU-resident affine weight after the load-time repack.
struct AffineWeight {
    Device *dev = nullptr;
    int N = 0, K = 0, group_size = 0, bits = 0, G = 0;
    uint8_t *codes = nullptr;  // [N, K/2] (4-bit) or [N, K] (8-bit), row-major, 16-byte aligned rows
    __half2 *sz = nullptr;     // [N, G] interleaved (scale, zero) fp16
    __half *awq = nullptr;     // [K] or nullptr
    // 4-bit, group 128: tiles of 16 rows x 128 columns (1 KB of nibbles) in [row block][group] order and
    // the 16 (scale, zero) pairs of each tile; see matvec_v2.cu
    uint8_t *tiles = nullptr;
    int nblk = 0;
    // gate+up pair in one tile stream (tile rows 0-7 from this matrix, 8-15 from `pair_with`), built on first use
    uint8_t *pair_tiles = nullptr;
    const AffineWeight *pair_with = nullptr;
    int pair_nblk = 0;
    size_t bytes = 0;
};

// bytes of one tile of the tile-major weight stream: 16 rows x 128 columns of codes + 16 (scale, zero) fp16 pairs
inline size_t tile_bytes_of(int bits) { return bits == 4 ? 1088 : 2112; }

struct V2Params {
    const uint8_t *tiles;  // [nblk][G][1088]: 1024 bytes of nibbles + 16 (scale, zero) pairs per tile
    const __half *awq, *x, *b, *gamma;
    __half *y, *residual_out, *normed_out;
    float eps;
    int N;       // logical outputs per batch row
    int K, G, nblk;
    int nring;   // stages in the shared-memory ring
    int split_tiles;  // 1: CTAs split the flattened tile list (stream-K); 0: whole row blocks per CTA
    float *partial;  // [grid][2][64]
    int *counters;   // [nblk], zero between launches
    int *err;
};

// INT4 g128 GEMM on tcgen05 / TMEM (gemm_tc.cu): y[M, N] = f16(x / awq) * dequant(w)^T; xs_scratch holds M * K halves.
// IM_ERR_BOUNDS when the weight is not INT4 group-128.
int gemm_affine_tc(const AffineWeight *w, const __half *x, __half *y, int M, __half *xs_scratch, cudaStream_t st);
// Gate/up pair as one tile stream (matvec.cu); built on first use.
int ensure_pair(const AffineWeight *gate, const AffineWeight *up, cudaStream_t st);
int v2_run(int mode, int nb, const V2Params &p, const Device *dev, cudaStream_t st, int bits = 4);
int v2_repack8(const uint8_t *codes, const __half2 *sz, int N, int K, int G, int nblk, uint8_t *tiles, cudaStream_t st);
int v2_repack(const uint8_t *codes0, const __half2 *sz0, const uint8_t *codes1, const __half2 *sz1, int N, int K, int G, int nblk,
              int rows_per_blk, uint8_t *tiles, cudaStream_t st);

// ---- programmatic dependent launch ------------------------------------------
// Decode is a chain of ~230 short kernels per token.  Launched with the programmatic-serialization
// attribute, a kernel may start while its predecessor is still draining: everything it does before
// pdl_wait() (barrier set-up, streaming constant weights into shared memory) overlaps the predecessor's
// tail; pdl_wait() returns once the predecessor has completed and its writes are visible.  Every kernel
// launched through launch_k() must therefore call pdl_wait() before it reads anything a predecessor wrote
// and before its first global write.

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// ---- device helpers -------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Streaming 128-bit load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
    uint4 r;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// 4-way byte dot products: unsigned codes against signed / unsigned activation bytes.
__device__ __forceinline__ int dp4a_us(unsigned a, unsigned b_signed, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b_signed), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(unsigned a, unsigned b, int c) {
    unsigned d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"((unsigned)c));
    return (int)d;
}

// Arguments of the fused (QK-norm +) RoPE kernel (norm.cu), shared with the model engine.
struct QkRopeArgs {
    const __half *q_in, *k_in, *v_in;
    int q_stride, k_stride, v_stride;  // elements between consecutive tokens of the inputs
    __half *q_out, *k_out, *v_out;
    const __half *qw, *kw, *cosc, *sinc;
    int nh, nkv, hd, rotary_dim, seq_offset;
    const int *pos_dev;  // per-sequence base positions (tokens_per_seq tokens each) or nullptr
    int tokens_per_seq;
    float eps;
    int with_norm;
};

int launch_qk_rope(const QkRopeArgs &a, int T, cudaStream_t st);

// TurboQuant constants + scratch (turboquant.cu)
struct Tq {
    Device *dev = nullptr;
    int hd = 0, n_bits = 0, k_levels = 0, v_levels = 0;
    float *signs = nullptr, *qjl = nullptr, *qjl_t = nullptr, *k_cb = nullptr, *k_bd = nullptr, *v_cb = nullptr, *v_bd = nullptr;
    float *scratch = nullptr;
    size_t scratch_bytes = 0;
    size_t const_bytes = 0;
};

int tq_auto_splits(const Device *dev, int nseq, int T, int nkv, int seq_len);
int tq_reduce_launch(const Tq *tq, const float *po, const float *pm, const float *pl, __half *out, int tokens, int nh, int splits, cudaStream_t st);
// Prefill chunks of one sequence: dequantise the cached rows once, causal flash attention on the tensor cores (tq_prefill.cu).
size_t tq_prefill_scratch_bytes(int nkv, int max_seq);
int tq_prefill_attention_launch(const Tq *tq, float *partials, void *dq, const float *qrot, const uint8_t *kc, const uint8_t *vc, const float *ks,
                                const float *vs, const float *krn, float attn_scale, __half *out, int slot, int nh, int nkv, int max_seq,
                                const int *pos_dev, int T, int ctx_end, cudaStream_t st, int base_pos = 0, bool project_queries = true);
bool tq_prefill_takes(int nh, int nkv);  // head groupings the prefill pass is built for
// Inputs of the fused RoPE + cache write + query rotation launch (turboquant.cu).
struct TqPrep {
    const __half *qkv;  // [nseq*T, stride]: q | k | v of one token
    int stride, k_off, v_off;
    const __half *kv = nullptr;  // optional: K and V rows live in their own buffer [nseq*T, kv_stride]; k_off / v_off index it
    int kv_stride = 0;
    const __half *qw, *kw, *cosc, *sinc;
    int nh, nkv, rotary_dim, with_norm, T, nseq, max_seq, base_pos;
    float eps;
    const int *pos_dev;
    const int *slot_map = nullptr;  // optional: sequence index -> cache slot
    float *qrot;    // out [nseq*T, nh, 2, hd]
    __half *q_out;  // optional out [nseq*T, nh, hd]
    uint8_t *kc, *vc;
    float *ks, *vs, *krn;
    int no_q_proj = 0;  // query heads: leave S * (rotated query) to the consumer (the prefill attention pass projects it itself)
};
int tq_prep_launch(const Tq *tq, const TqPrep &a, cudaStream_t st);
int tq_attention_launch(const Tq *tq, float *scratch, const __half *q, const uint8_t *kc, const uint8_t *vc, const float *ks,
                        const float *vs, const float *krn, float attn_scale, __half *out, int nseq, int nh, int nkv, int max_seq,
                        int base_pos, const int *pos_dev, int T, int splits, cudaStream_t st, const float *qrot = nullptr,
                        const int *slot_map = nullptr);

// ---- fp16 (unquantized) KV cache: kv_f16.cu ----
struct Kv16Prep {
    __half *qkv;  // [nseq*T, stride]: q | k | v of one token; the query heads are normed / rotated in place
    int stride, k_off, v_off;
    const __half *kv;  // nullptr, or the buffer [nseq*T, kv_stride] that holds the K and V rows (k_off / v_off index it)
    int kv_stride;
    const __half *qw, *kw, *cosc, *sinc;
    int nh, nkv, rotary_dim, with_norm, T, nseq, max_seq, base_pos;
    float eps;
    const int *pos_dev;
    const int *slot_map;  // optional: sequence index -> cache slot
    __half *kc, *vc;      // [slots, nkv, max_seq, 128]
};
int kv16_prep_launch(const Kv16Prep &a, cudaStream_t st);
size_t kv16_scratch_bytes(int tokens, int nh, int splits);
int kv16_auto_splits(const Device *dev, int tokens, int nkv, int max_ctx);
int kv16_attention_launch(const Device *dev, float *scratch, size_t scratch_bytes, const __half *q, int q_stride, const __half *kc, const __half *vc,
                          float scale, __half *out, int nseq, int nh, int nkv, int max_seq, int base_pos, const int *pos_dev, int T, int splits,
                          int ctx_hint, cudaStream_t st, const int *slot_map, int prefill_slot = -1);  // prefill_slot >= 0: one sequence in that cache slot

}  // namespace im

// The opaque handle types of the C ABI are thin tags over the internal structs.
struct im_device : im::Device {};
struct im_affine_weight : im::AffineWeight {};
