// Model-level decode engine: the CUDA counterpart of MetalInference
// (crates/ironmill-inference/src/metal/engine.rs:122-270, loading.rs:32-518, pipeline.rs:228-1313).
//
// Schedule of one token (pipeline.rs:424-1313, decode DAG metal/graph.rs:98-201):
//   fused_embedding_norm -> per layer { QKV projection (layer 0; later layers get it from the
//   end-of-layer fused kernel), (QK-norm +) RoPE, TurboQuant write of K and V, TurboQuant split
//   attention + reduce, o_proj, fused residual+RMSNorm, fused gate+up+SiLU, down_proj, fused
//   residual+RMSNorm+next-layer QKV projection } -> final RMSNorm -> fp16 lm_head.
// The whole step is captured once per batch size into a CUDA graph; the sequence position lives
// in device memory so that the graph replays unchanged as the sequence grows.
//
// Tensor parallelism (not present in the reference): QKV / gate / up are split by output rows
// (heads), o / down by input columns, KV heads and their caches by rank, lm_head by vocabulary
// rows; one NCCL all-reduce follows each row-split projection and one all-gather the lm_head.
#include <dlfcn.h>
#include <math.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"
#include "mega.cuh"
#if defined(__x86_64__)
#include <immintrin.h>
#endif

#if __has_include(<nccl.h>)
#include <nccl.h>
#define IM_HAVE_NCCL_H 1
#else
#define IM_HAVE_NCCL_H 0
#endif

// entry points of other translation units used here
extern "C" {
struct im_tq;
int im_cuda_tq_generate(int head_dim, uint64_t seed, float *signs_out_host, float *qjl_out_host);
int im_cuda_tq_create(im_device *dev, int head_dim, int n_bits, const float *signs_host, const float *qjl_host,
                      const float *k_levels_host, const float *k_bounds_host, const float *v_levels_host,
                      const float *v_bounds_host, im_tq **out);
void im_cuda_tq_free(im_tq *tq);
int im_cuda_tq_encode(const im_tq *tq, const void *kv_dev, int is_k, void *cache_dev, float *scale_dev, float *r_norms_dev,
                      int nseq, int nkv, int max_seq, int base_pos, const int *pos_dev, int T, void *stream);
size_t im_cuda_tq_scratch_bytes(int nseq, int T, int nh, int head_dim, int splits);
int im_cuda_tq_reserve_scratch(im_tq *tq, size_t bytes);
}

namespace im {

// ---- NCCL through dlopen: the library works without NCCL until tensor parallelism is asked for
#if IM_HAVE_NCCL_H
struct Nccl {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
static Nccl *nccl() {
    static Nccl n;
    static bool tried = false;
    if (!tried) {
        tried = true;
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            n.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (n.lib) break;
        }
        if (n.lib) {
#define IM_SYM(field, sym) n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.lib, sym))
            IM_SYM(GetUniqueId, "ncclGetUniqueId");
            IM_SYM(CommInitRank, "ncclCommInitRank");
            IM_SYM(AllReduce, "ncclAllReduce");
            IM_SYM(AllGather, "ncclAllGather");
            IM_SYM(CommDestroy, "ncclCommDestroy");
            IM_SYM(GetErrorString, "ncclGetErrorString");
#undef IM_SYM
        }
    }
    return (n.lib && n.GetUniqueId && n.CommInitRank && n.AllReduce && n.AllGather) ? &n : nullptr;
}
#define IM_NCCL_CHECK(expr)                                                                              \
    do {                                                                                                 \
        ncclResult_t _r = (expr);                                                                        \
        if (_r != ncclSuccess)                                                                           \
            return fail(IM_ERR_NCCL, "%s failed: %s", #expr, nccl()->GetErrorString ? nccl()->GetErrorString(_r) : "?"); \
    } while (0)
#endif

struct HostAffine {  // one projection as handed to load_affine, already cut to this rank's shard
    std::vector<uint8_t> q;
    std::vector<float> s, z;  // kept as f32 or widened fp16 bit patterns, see param_f32
    std::vector<uint16_t> s16, z16, awq;
    bool param_f32 = true, have = false;
    int N = 0, K = 0, gs = 0, bits = 0;
};

// ---- one-shot all-reduce over peer memory (tensor parallel, small vectors) --------------------------------
// A decode step has two row-split projections per layer, each followed by a sum of a [batch, hidden] fp16 vector over
// the ranks: 8 KB at batch 1, 65 times per token.  NCCL's all-reduce costs 15-30 us there, more than the projections.
// Here every rank stores its vector into a slot of EVERY rank's receive buffer (plain stores to peer memory over
// NVLink), raises a per-source sequence flag on every rank, waits (bounded) until all sources have raised theirs, and
// sums the world's vectors from its own memory in rank order, in f32, rounding once.  Two buffer halves alternate:
// a rank can only be one all-reduce ahead of the slowest one.  Plain peer stores only: nothing goes through the
// switch's reduction or replication units.
constexpr int kXarMaxWorld = 8, kXarThreads = 512;
struct PeerAllreduce {
    bool ok = false;
    unsigned char *base = nullptr;  // this rank's allocation: [flags: kXarMaxWorld u32][seq u32][pad to 256][buf: 2 x world x cap halves]
    size_t bytes = 0, cap = 0;      // cap: halves per vector
    unsigned char *peer[kXarMaxWorld] = {};  // every rank's allocation as mapped here (own included)
    // appended for the tensor-parallel whole-token kernel: [mailboxes: 4 x world x hidden/2 x {2 halves, tag}][launch count]
    size_t mail_off = 0, epoch_off = 0;
};
struct XarArgs {
    unsigned *flags, *seq;             // local
    __half *buf;                       // local receive buffer
    unsigned *peer_flags[kXarMaxWorld];
    __half *peer_buf[kXarMaxWorld];
    int world, rank;
    size_t cap;
    int *err;
};
__global__ void __launch_bounds__(kXarThreads) peer_allreduce_kernel(const XarArgs x, const __half *__restrict__ in, __half *__restrict__ out,
                                                                      int count) {
    __shared__ int s_ok;
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, chunks = count / 8;
    const unsigned seq = *x.seq + 1u;
    const size_t slot = (size_t)(seq & 1u) * x.world;
    for (int c = tid; c < chunks; c += kXarThreads) {
        const uint4 v = reinterpret_cast<const uint4 *>(in)[c];
        for (int p = 0; p < x.world; p++) reinterpret_cast<uint4 *>(x.peer_buf[p] + (slot + x.rank) * x.cap)[c] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) s_ok = 1;
    if (tid < x.world) {
        __threadfence_system();
        *reinterpret_cast<volatile unsigned *>(x.peer_flags[tid] + x.rank) = seq;  // "my vector number seq is in your buffer"
    }
    __syncthreads();
    if (tid < x.world) {  // one poller per source; sequence numbers only grow
        const volatile unsigned *f = x.flags + tid;
        unsigned long long t0 = 0;
        for (unsigned i = 0;; i++) {
            if ((int)(*f - seq) >= 0) break;
            if ((i & 255u) == 255u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                // ranks are separate processes whose hosts may lag each other by a scheduling hiccup: 5 s before a rank is
                // given up; once the error word is set no later all-reduce waits at all
                if (now - t0 > 5000ull * 1000 * 1000 || *reinterpret_cast<volatile int *>(x.err) != 0) {
                    atomicExch(x.err, 3);
                    s_ok = 0;
                    break;
                }
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    if (s_ok) {
        for (int c = tid; c < chunks; c += kXarThreads) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int p = 0; p < x.world; p++) {
                const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x.buf + (slot + p) * x.cap) + c);
                const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(h[i]);
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                }
            }
            uint4 r;
            __half2 *hr = reinterpret_cast<__half2 *>(&r);
#pragma unroll
            for (int i = 0; i < 4; i++) hr[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
            reinterpret_cast<uint4 *>(out)[c] = r;
        }
    }
    if (tid == 0) *x.seq = seq;
}

struct Layer {
    HostAffine hq, hk, hv;           // staged until finalize concatenates them
    AffineWeight *qkv = nullptr;     // rows [q | k | v] of this rank
    AffineWeight q_rows{}, kv_rows{};  // non-owning views of qkv's Q rows and K | V rows (same device arrays)
    AffineWeight *o = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
    __half *input_ln = nullptr, *post_ln = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    uint8_t *kc = nullptr, *vc = nullptr;
    float *ks = nullptr, *vs = nullptr, *krn = nullptr;
};

struct Model {
    Device *dev = nullptr;
    im_model_config cfg{};
    int nh_l = 0, nkv_l = 0, I_l = 0, vocab_l = 0, world = 1, rank = 0;
    int q_dim = 0, kv_dim = 0, qkv_dim = 0;
    std::vector<Layer> layers;
    __half *embed = nullptr, *lm_head = nullptr, *final_norm = nullptr;
    bool lm_head_owned = false;
    im_tq *tq = nullptr;
    std::vector<float> signs_host, qjl_host;
    __half *cosc = nullptr, *sinc = nullptr;
    // activations, MT = max tokens per forward
    int MT = 0;
    __half *hidden = nullptr, *norm_out = nullptr, *residual = nullptr, *qkv = nullptr, *q_d = nullptr, *k_d = nullptr,
           *attn_out = nullptr, *ffn_down = nullptr, *ffn_gate = nullptr, *ffn_up = nullptr, *xs_scratch = nullptr, *logits = nullptr,
           *logits_all = nullptr;
    bool gemm_ok = false;  // every projection is INT4 or INT8 group-128: forwards of 16 tokens and more run the tensor-core GEMM
    float *qrot = nullptr;  // [MT, nh_l, 2, hd] rotated queries
    uint32_t *tokens_dev = nullptr, *tok_hist = nullptr;
    int *pos_dev = nullptr, *step_dev = nullptr;
    uint32_t *tokens_pin = nullptr;
    __half *logits_pin = nullptr;
    float2 *argmax_cand = nullptr;  // [max_batch][kArgmaxCtas] candidates of the greedy pick
    unsigned *argmax_counters = nullptr;
    int *err_pin = nullptr;  // the device's bounded-wait error word, copied back with every step
    cudaStream_t stream = nullptr;
    std::map<int, cudaGraphExec_t> graphs;
    // Cache slots (continuous batching): every sequence owns one of max_batch slots = its rows of every layer's caches
    // and its position.  The single-sequence calls work on slot 0, the lockstep batch calls on slots 0 .. batch - 1.
    std::vector<int> slot_pos;      // host copy of the positions
    std::vector<char> slot_used;    // claimed by im_cuda_model_seq_add
    int *slot_ident = nullptr;      // device: 0, 1, 2, ... (a one-sequence forward into slot s passes slot_ident + s)
    int *slot_map = nullptr;        // device: slots of the sequences of the batch being decoded
    int *slot_pin = nullptr;
    bool finalized = false;
    size_t bytes = 0;
    int launches_per_step = 0;
    float *scratch_ref = nullptr;
    void *pf_dq = nullptr;          // dequantised K' / V' rows of one sequence for prefill chunks (tq_prefill.cu)
    int prefill_slot_id = -1, prefill_ctx_end = 0;  // set around a prefill chunk's forward: the slot and its positions after the chunk
    float *kv16_scratch = nullptr;  // split partials of the fp16-KV attention (tq_bits == 16)
    size_t kv16_scratch_bytes = 0;
    // whole-token decode kernel (batch 1, single GPU): tables built by mega_prepare()
    bool mega_ready = false;
    MegaParams mega{};
    bool mega_capacity2 = false;  // one GPU, tagged hand-over: mailboxes sized for one more (missing) rank (test hook)
    uint2 *mega_phantom_mail = nullptr;
    __half *logits_seq = nullptr;  // [prefill chunk, vocab_l] logits of every token (prefill_all_logits), allocated on first use
    __half *logits_seq_all = nullptr;
    __half *logits_seq_pin = nullptr;
#if IM_HAVE_NCCL_H
    ncclComm_t comm = nullptr;
#endif
    PeerAllreduce xar;
    std::vector<std::pair<void *, size_t>> allocs;

    int alloc(void **p, size_t n) {
        int rc = dev_malloc(dev, p, n);
        if (rc == IM_OK && n) {
            allocs.push_back({*p, n});
            bytes += n;
        }
        return rc;
    }
};

// Tokens per prefill forward: the tensor-core GEMMs fill the GPU from about a thousand tokens on (a 256-token chunk is
// 32-112 CTAs per projection), so the default is the largest chunk; the activation buffers are sized for the configured
// chunk (at most max_seq_len).  prefill_all_logits keeps 256-token chunks: it holds a chunk's logits for every token.
static const int kPrefillChunk = 2048;
static const int kAllLogitsChunk = 256;
static const int kGemmMinTokens = 16;  // from here on the projections are dense contractions: tcgen05 GEMM instead of matvecs

__global__ void advance_pos_kernel(int *pos, const int *slot_map, int n, int by) {
    pdl_trigger();
    pdl_wait();
    if ((int)threadIdx.x < n) pos[slot_map ? slot_map[threadIdx.x] : threadIdx.x] += by;
}
__global__ void set_pos_kernel(int *pos, int n, int v) {
    if ((int)threadIdx.x < n) pos[threadIdx.x] = v;
}

// Greedy pick per sequence: LAST maximal index (Iterator::max_by keeps the last of equal maxima,
// crates/ironmill-inference/src/sampling.rs:331-339).  logits are laid out [parts][nseq][vocab_part].
// grid (kArgmaxCtas, nseq): every CTA scans a slice of the vocabulary and leaves its candidate in `cand`; the last
// CTA of a sequence to arrive combines the candidates, writes the token and clears the counter for the next launch.
constexpr int kArgmaxCtas = 64, kArgmaxThreads = 256;
__device__ __forceinline__ bool argmax_better(float ov, int oi, float best, int bi) {  // is (ov, oi) preferred over (best, bi)?
    return oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi));
}
__global__ void __launch_bounds__(kArgmaxThreads) argmax_kernel(const __half *__restrict__ logits, int vocab_part, int parts, int nseq,
                                                                uint32_t *__restrict__ tokens, uint32_t *__restrict__ hist,
                                                                const int *__restrict__ step, int hist_stride, int hist_rows,
                                                                float2 *__restrict__ cand, unsigned *__restrict__ counters) {
    __shared__ float sv[kArgmaxThreads / 32];
    __shared__ int si[kArgmaxThreads / 32];
    __shared__ int s_last;
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y;
    const int vocab = vocab_part * parts;
    const int per = (vocab + gridDim.x - 1) / gridDim.x, i0 = blockIdx.x * per, i1 = min(vocab, i0 + per);
    float best = -INFINITY;
    int bi = -1;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const int part = i / vocab_part, j = i % vocab_part;
        const float v = __half2float(logits[((size_t)part * nseq + seq) * vocab_part + j]);
        if (!(v < best) || bi < 0) {  // ascending i per thread: ties move to the later index
            best = v;
            bi = i;
        }
    }
    auto block_reduce = [&]() {
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (argmax_better(ov, oi, best, bi)) {
                best = ov;
                bi = oi;
            }
        }
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (lane == 0) {
            sv[warp] = best;
            si[warp] = bi;
        }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int w = 1; w < (int)(blockDim.x >> 5); w++)
                if (argmax_better(sv[w], si[w], best, bi)) {
                    best = sv[w];
                    bi = si[w];
                }
    };
    block_reduce();
    if (threadIdx.x == 0) {
        cand[(size_t)seq * gridDim.x + blockIdx.x] = make_float2(best, __int_as_float(bi));
        __threadfence();
        s_last = atomicAdd(&counters[seq], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = -INFINITY;
    bi = -1;
    if (threadIdx.x < gridDim.x) {
        const float2 c = __ldcg(&cand[(size_t)seq * gridDim.x + threadIdx.x]);
        best = c.x;
        bi = __float_as_int(c.y);
    }
    __syncthreads();
    block_reduce();
    if (threadIdx.x == 0) {
        tokens[seq] = (uint32_t)bi;
        if (hist) hist[(size_t)(*step % hist_rows) * hist_stride + seq] = (uint32_t)bi;
        counters[seq] = 0;
    }
}
__global__ void bump_kernel(int *step) {
    pdl_trigger();
    pdl_wait();
    *step += 1;
}

// act[i] = SiLU(gate[i]) * up[i] (crates/ironmill-inference/src/metal/shaders/activation/activation.metal silu_gate), f32 inside
__global__ void silu_mul_kernel(const __half *__restrict__ gate, const __half *__restrict__ up, __half *__restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    const float2 g = __half22float2(*reinterpret_cast<const __half2 *>(gate + i)), u = __half22float2(*reinterpret_cast<const __half2 *>(up + i));
    *reinterpret_cast<__half2 *>(out + i) = __floats2half2_rn((g.x / (1.0f + expf(-g.x))) * u.x, (g.y / (1.0f + expf(-g.y))) * u.y);
}

}  // namespace im
// silu_gate as an entry point of its own (the prefill form of the FFN: gate and up are rounded to fp16 first).
// out may alias gate.  n even.
IM_EXPORT int im_cuda_silu_mul(const void *gate_dev, const void *up_dev, void *out_dev, size_t n, void *stream) {
    IM_GUARD_BEGIN
    IM_REQUIRE(gate_dev && up_dev && out_dev && n % 2 == 0, "bad argument");
    if (n == 0) return IM_OK;
    cudaError_t le = im::launch_k(im::silu_mul_kernel, dim3((unsigned)((n / 2 + 255) / 256)), dim3(256), 0, im::as_stream(stream),
                                  static_cast<const __half *>(gate_dev), static_cast<const __half *>(up_dev), static_cast<__half *>(out_dev), n);
    if (le != cudaSuccess) return im::fail(IM_ERR_CUDA, "launch failed: %s", cudaGetErrorString(le));
    return IM_OK;
    IM_GUARD_END
}
namespace im {

static bool parse_layer_name(const char *name, int *layer, std::string *suffix) {
    const char *pfx = "model.layers.";
    if (strncmp(name, pfx, strlen(pfx)) != 0) return false;
    const char *p = name + strlen(pfx);
    char *end = nullptr;
    long l = strtol(p, &end, 10);
    if (end == p || *end != '.') return false;
    *layer = (int)l;
    *suffix = end + 1;
    return true;
}

static int upload_f16(Model *m, __half **dst, const void *src, size_t n) {
    int rc = m->alloc((void **)dst, n * sizeof(__half));
    if (rc != IM_OK) return rc;
    IM_CUDA_CHECK(cudaMemcpy(*dst, src, n * sizeof(__half), cudaMemcpyHostToDevice));
    return IM_OK;
}

// The rectangle of a full projection that a tensor-parallel rank keeps: q/k/v/gate/up are split by output rows
// (whole heads), o/down by input columns; (en, ek) is the full shape the tensor must have.
static int shard_rect(const im_model_config &c, const std::string &suffix, int *r0, int *nr, int *c0, int *nc, int *en, int *ek) {
    const int world = c.tp_world > 0 ? c.tp_world : 1, r = c.tp_rank, H = c.hidden_size, hd = c.head_dim;
    const int q_dim = c.num_heads / world * hd, kv_dim = c.num_kv_heads / world * hd, I_l = c.intermediate_size / world;
    if (suffix == "self_attn.q_proj.weight") { *en = c.num_heads * hd; *ek = H; *r0 = r * q_dim; *nr = q_dim; *c0 = 0; *nc = H; }
    else if (suffix == "self_attn.k_proj.weight" || suffix == "self_attn.v_proj.weight") { *en = c.num_kv_heads * hd; *ek = H; *r0 = r * kv_dim; *nr = kv_dim; *c0 = 0; *nc = H; }
    else if (suffix == "self_attn.o_proj.weight") { *en = H; *ek = c.num_heads * hd; *r0 = 0; *nr = H; *c0 = r * q_dim; *nc = q_dim; }
    else if (suffix == "mlp.gate_proj.weight" || suffix == "mlp.up_proj.weight") { *en = c.intermediate_size; *ek = H; *r0 = r * I_l; *nr = I_l; *c0 = 0; *nc = H; }
    else if (suffix == "mlp.down_proj.weight") { *en = H; *ek = c.intermediate_size; *r0 = 0; *nr = H; *c0 = r * I_l; *nc = I_l; }
    else return IM_ERR_INVALID;
    return IM_OK;
}

// Cut rows [r0, r0+nr) and columns [c0, c0+nc) out of a full affine tensor.
static int slice_affine(HostAffine *out, const void *qdata, const void *scales, const void *zeros, int param_dtype, const void *awq,
                        int N, int K, int gs, int bits, int r0, int nr, int c0, int nc) {
    if (r0 < 0 || nr <= 0 || r0 + nr > N || c0 < 0 || nc <= 0 || c0 + nc > K) return fail(IM_ERR_INVALID, "shard out of range");
    if ((c0 % gs) != 0 || (nc % gs != 0 && c0 + nc != K) || (bits == 4 && ((c0 | nc | K) & 1)))
        return fail(IM_ERR_INVALID, "column shard [%d,%d) of K=%d is not aligned to group size %d", c0, c0 + nc, K, gs);
    const int G = (K + gs - 1) / gs, g0 = c0 / gs, ng = (nc + gs - 1) / gs;
    const size_t rb = (size_t)K * bits / 8, cb0 = (size_t)c0 * bits / 8, cbn = (size_t)nc * bits / 8;
    out->N = nr; out->K = nc; out->gs = gs; out->bits = bits; out->have = true;
    out->param_f32 = param_dtype == IM_DTYPE_F32;
    out->q.resize((size_t)nr * cbn);
    const uint8_t *q = static_cast<const uint8_t *>(qdata);
    for (int r = 0; r < nr; r++) memcpy(out->q.data() + (size_t)r * cbn, q + (size_t)(r0 + r) * rb + cb0, cbn);
    if (out->param_f32) {
        out->s.resize((size_t)nr * ng);
        out->z.resize((size_t)nr * ng);
        for (int r = 0; r < nr; r++) {
            memcpy(out->s.data() + (size_t)r * ng, static_cast<const float *>(scales) + (size_t)(r0 + r) * G + g0, ng * 4);
            memcpy(out->z.data() + (size_t)r * ng, static_cast<const float *>(zeros) + (size_t)(r0 + r) * G + g0, ng * 4);
        }
    } else {
        out->s16.resize((size_t)nr * ng);
        out->z16.resize((size_t)nr * ng);
        for (int r = 0; r < nr; r++) {
            memcpy(out->s16.data() + (size_t)r * ng, static_cast<const uint16_t *>(scales) + (size_t)(r0 + r) * G + g0, ng * 2);
            memcpy(out->z16.data() + (size_t)r * ng, static_cast<const uint16_t *>(zeros) + (size_t)(r0 + r) * G + g0, ng * 2);
        }
    }
    out->awq.clear();
    if (awq) out->awq.assign(static_cast<const uint16_t *>(awq) + c0, static_cast<const uint16_t *>(awq) + c0 + nc);
    return IM_OK;
}

static int make_weight(Model *m, const HostAffine &h, AffineWeight **out) {
    im_affine_weight *w = nullptr;
    int rc = im_cuda_affine_weight_create(static_cast<im_device *>(m->dev), h.q.data(), h.param_f32 ? (const void *)h.s.data() : (const void *)h.s16.data(),
                                          h.param_f32 ? (const void *)h.z.data() : (const void *)h.z16.data(),
                                          h.param_f32 ? IM_DTYPE_F32 : IM_DTYPE_F16, h.awq.empty() ? nullptr : h.awq.data(), h.N, h.K, h.gs,
                                          h.bits, &w);
    if (rc != IM_OK) return rc;
    *out = w;
    m->bytes += w->bytes;
    return IM_OK;
}

// Rows [row0, row0 + rows) of a weight as a weight of its own (non-owning; row0 a multiple of 16 so that the tiled
// stream splits between row blocks).
static AffineWeight row_view(const AffineWeight *w, int row0, int rows) {
    AffineWeight v = *w;
    v.N = rows;
    v.codes = w->codes ? w->codes + (size_t)row0 * ((size_t)w->K * w->bits / 8) : nullptr;
    v.sz = w->sz ? w->sz + (size_t)row0 * w->G : nullptr;
    v.tiles = w->tiles ? w->tiles + (size_t)(row0 / 16) * w->G * tile_bytes_of(w->bits) : nullptr;
    v.nblk = (rows + 15) / 16;
    v.pair_tiles = nullptr;
    v.pair_with = nullptr;
    v.pair_nblk = 0;
    v.bytes = 0;
    return v;
}

static int tp_allreduce(Model *m, __half *buf, size_t count, cudaStream_t st) {
    if (m->world <= 1) return IM_OK;
#if IM_HAVE_NCCL_H
    if (!m->comm) return fail(IM_ERR_STATE, "tensor parallel group not initialised (im_cuda_model_tp_init)");
    if (m->xar.ok && count <= m->xar.cap && count % 8 == 0) {
        XarArgs x{};
        x.flags = reinterpret_cast<unsigned *>(m->xar.base);
        x.seq = x.flags + kXarMaxWorld;
        x.buf = reinterpret_cast<__half *>(m->xar.base + 256);
        for (int p = 0; p < m->world; p++) {
            x.peer_flags[p] = reinterpret_cast<unsigned *>(m->xar.peer[p]);
            x.peer_buf[p] = reinterpret_cast<__half *>(m->xar.peer[p] + 256);
        }
        x.world = m->world; x.rank = m->rank; x.cap = m->xar.cap; x.err = m->dev->err_flag;
        IM_CUDA_CHECK(launch_k(peer_allreduce_kernel, dim3(1), dim3(kXarThreads), 0, st, x, (const __half *)buf, buf, (int)count));
        return IM_OK;
    }
    IM_NCCL_CHECK(nccl()->AllReduce(buf, buf, count, ncclHalf, ncclSum, m->comm, st));
    return IM_OK;
#else
    (void)buf; (void)count; (void)st;
    return fail(IM_ERR_NCCL, "built without nccl.h");
#endif
}

// Per-category GPU timing of one eager step (the counterpart of MetalConfig.kernel_timing /
// the profile-metal feature, crates/ironmill-inference/src/metal/pipeline.rs:353-422,1215-1234):
// an event is recorded after each group of launches and the interval is charged to its category.
enum ProfCat { kCatEmbed = 0, kCatQkv, kCatRope, kCatKvWrite, kCatAttn, kCatOProj, kCatResNorm, kCatFfn, kCatDown, kCatComm, kCatHead, kCatCount };
struct Prof {
    cudaStream_t st;
    std::vector<cudaEvent_t> ev;
    std::vector<int> cat;
    void mark(int c) {
        cudaEvent_t e;
        cudaEventCreate(&e);
        cudaEventRecord(e, st);
        ev.push_back(e);
        cat.push_back(c);
    }
};
#define IM_MARK(c) do { if (prof) prof->mark(c); } while (0)

#define IM_TRY(expr)                  \
    do {                              \
        int _rc = (expr);             \
        if (_rc != IM_OK) return _rc; \
    } while (0)

// One forward pass over nseq sequences x T tokens each (decode: T = 1; prefill: nseq = 1).
// Logits are produced for the last token of every sequence.
// slots: device array naming the cache slot of each of the nseq sequences (nullptr: slots 0 .. nseq - 1).
// (QK-norm +) RoPE, cache write and attention of one layer.  TurboQuant caches: the fused preparation (cache write
// and query rotation), split attention, reduction.  fp16 cache (TurboQuant off): norm / RoPE in place, the K / V rows
// scattered as fp16, one attention kernel over the fp16 rows (kv_f16.cu).  q_buf: the buffer a.qkv names, writable.
// part 0: the preparation (cache write), part 1: the attention.
static int attention_block(Model *m, int part, const TqPrep &a, __half *q_buf, Layer &L, int nseq, int T, float attn_scale, int attn_splits,
                           const int *slots, cudaStream_t st) {
    const im_model_config &c = m->cfg;
    if (c.tq_bits == 16) {
        Kv16Prep k{};
        k.qkv = q_buf; k.stride = a.stride; k.k_off = a.k_off; k.v_off = a.v_off; k.kv = a.kv; k.kv_stride = a.kv_stride;
        k.qw = a.qw; k.kw = a.kw; k.cosc = a.cosc; k.sinc = a.sinc; k.nh = a.nh; k.nkv = a.nkv; k.rotary_dim = a.rotary_dim;
        k.with_norm = a.with_norm; k.T = T; k.nseq = nseq; k.max_seq = a.max_seq; k.base_pos = 0; k.eps = a.eps; k.pos_dev = a.pos_dev;
        k.slot_map = slots; k.kc = reinterpret_cast<__half *>(L.kc); k.vc = reinterpret_cast<__half *>(L.vc);
        if (part == 0) return kv16_prep_launch(k, st);
        return kv16_attention_launch(m->dev, m->kv16_scratch, m->kv16_scratch_bytes, q_buf, a.stride, k.kc, k.vc, attn_scale, m->attn_out, nseq, a.nh,
                                     a.nkv, c.max_seq_len, 0, m->pos_dev, T, 0, c.max_seq_len, st, slots, nseq == 1 ? m->prefill_slot_id : -1);
    }
    // a prefill chunk of one sequence: dequantise the cached rows once, causal tensor-core pass (which also projects the queries)
    const bool flash = nseq == 1 && T >= 16 && m->pf_dq && m->prefill_slot_id >= 0 && tq_prefill_takes(a.nh, a.nkv);
    if (part == 0) {
        TqPrep b = a;
        b.no_q_proj = flash ? 1 : 0;
        return tq_prep_launch(reinterpret_cast<const Tq *>(m->tq), b, st);
    }
    if (flash) {
        const int rc = tq_prefill_attention_launch(reinterpret_cast<const Tq *>(m->tq), m->scratch_ref, m->pf_dq, m->qrot, L.kc, L.vc, L.ks, L.vs, L.krn,
                                                   attn_scale, m->attn_out, m->prefill_slot_id, a.nh, a.nkv, c.max_seq_len, m->pos_dev, T,
                                                   m->prefill_ctx_end, st);
        if (rc != IM_ERR_BOUNDS) return rc;  // head groupings it does not take: the per-token kernel below
    }
    return tq_attention_launch(reinterpret_cast<const Tq *>(m->tq), m->scratch_ref, nullptr, L.kc, L.vc, L.ks, L.vs, L.krn, attn_scale, m->attn_out,
                               nseq, a.nh, a.nkv, c.max_seq_len, 0, m->pos_dev, T, attn_splits, st, m->qrot, slots);
}

static int forward(Model *m, int nseq, int T, int attn_splits, cudaStream_t st, int *launches, Prof *prof = nullptr, bool all_logits = false,
                   const int *slots = nullptr) {
    const im_model_config &c = m->cfg;
    const int H = c.hidden_size, hd = c.head_dim, MT = nseq * T;
    const float eps = c.rms_eps;
    const float attn_scale = c.attn_scale != 0.0f ? c.attn_scale : 1.0f / sqrtf((float)hd);
    int nl = 0;
    IM_TRY(im_cuda_embedding_norm(m->tokens_dev, m->embed, m->layers[0].input_ln, m->norm_out, m->hidden, H, MT, (uint32_t)c.vocab_size, eps,
                                  c.embed_scale != 0.0f ? c.embed_scale : 1.0f, st));
    nl++;
    IM_MARK(kCatEmbed);
    const bool mega = MT == 1 && m->mega_ready && !prof && !slots;  // the whole-token kernel works on slot 0
    if (mega) {  // every layer in one persistent launch (decode_mega.cu); leaves the same buffers as the loop below
        int rc = mega_launch(m->mega, m->dev, st);
        if (rc == IM_ERR_BOUNDS) return fail(IM_ERR_INVALID, "whole-token decode kernel: shapes do not fit");
        IM_TRY(rc);
        IM_TRY(tp_allreduce(m, m->ffn_down, (size_t)H, st));  // tensor parallel: the last layer's down projection
        IM_TRY(im_cuda_residual_add(m->residual, m->ffn_down, m->hidden, (size_t)H, st));
        nl += 2 + (m->world > 1 ? 1 : 0);
    }
    // More than one token per sequence is the reference's prefill form (its matmul kernels round x / awq and the
    // dequantised weights to fp16: affine_matmul.metal:44-74), whatever the count; so are decode batches of 16 and more.
    const bool gemm = !mega && m->gemm_ok && (T > 1 || MT >= kGemmMinTokens);
    for (int l = 0; l < c.num_layers && gemm; l++) {
        // Dense contraction (prefill chunks, large decode batches): every projection is one tcgen05 GEMM; norms, SiLU
        // and the residual adds are separate element-wise launches (their bytes are a rounding error next to the GEMMs).
        Layer &L = m->layers[l];
        if (l == 0) {
            IM_TRY(gemm_affine_tc(L.qkv, m->norm_out, m->qkv, MT, m->xs_scratch, st));
            nl += 2;
            IM_MARK(kCatQkv);
        }
        TqPrep a{};
        a.qkv = m->qkv; a.stride = m->qkv_dim; a.k_off = m->q_dim; a.v_off = m->q_dim + m->kv_dim;
        a.qw = L.q_norm; a.kw = L.k_norm; a.cosc = m->cosc; a.sinc = m->sinc;
        a.nh = m->nh_l; a.nkv = m->nkv_l; a.rotary_dim = c.rotary_dim ? c.rotary_dim : hd; a.with_norm = c.qk_norm ? 1 : 0;
        a.T = T; a.nseq = nseq; a.max_seq = c.max_seq_len; a.base_pos = 0; a.eps = eps; a.pos_dev = m->pos_dev; a.slot_map = slots;
        a.qrot = m->qrot; a.q_out = nullptr;
        a.kc = L.kc; a.vc = L.vc; a.ks = L.ks; a.vs = L.vs; a.krn = L.krn;
        IM_TRY(attention_block(m, 0, a, m->qkv, L, nseq, T, attn_scale, attn_splits, slots, st));
        IM_MARK(kCatKvWrite);
        IM_TRY(attention_block(m, 1, a, m->qkv, L, nseq, T, attn_scale, attn_splits, slots, st));
        nl += 3;
        IM_MARK(kCatAttn);
        IM_TRY(gemm_affine_tc(L.o, m->attn_out, m->ffn_down, MT, m->xs_scratch, st));
        IM_MARK(kCatOProj);
        IM_TRY(tp_allreduce(m, m->ffn_down, (size_t)MT * H, st));  // tensor parallel: o is row-split
        if (m->world > 1) IM_MARK(kCatComm);
        IM_TRY(im_cuda_fused_residual_rms_norm(m->hidden, m->ffn_down, L.post_ln, m->norm_out, m->residual, H, MT, eps, st));
        IM_MARK(kCatResNorm);
        IM_TRY(gemm_affine_tc(L.gate, m->norm_out, m->ffn_gate, MT, m->xs_scratch, st));
        IM_TRY(gemm_affine_tc(L.up, m->norm_out, m->ffn_up, MT, m->xs_scratch, st));
        {
            const size_t n = (size_t)MT * m->I_l;
            cudaError_t le = launch_k(silu_mul_kernel, dim3((unsigned)((n / 2 + 255) / 256)), dim3(256), 0, st, (const __half *)m->ffn_gate,
                                      (const __half *)m->ffn_up, m->ffn_gate, n);
            if (le != cudaSuccess) return fail(IM_ERR_CUDA, "launch failed: %s", cudaGetErrorString(le));
        }
        IM_MARK(kCatFfn);
        IM_TRY(gemm_affine_tc(L.down, m->ffn_gate, m->ffn_down, MT, m->xs_scratch, st));
        IM_MARK(kCatDown);
        IM_TRY(tp_allreduce(m, m->ffn_down, (size_t)MT * H, st));  // tensor parallel: down is row-split
        if (m->world > 1) IM_MARK(kCatComm);
        nl += 11 + (m->world > 1 ? 2 : 0);
        if (l + 1 < c.num_layers) {
            Layer &Nx = m->layers[l + 1];
            IM_TRY(im_cuda_fused_residual_rms_norm(m->residual, m->ffn_down, Nx.input_ln, m->norm_out, m->hidden, H, MT, eps, st));
            IM_TRY(gemm_affine_tc(Nx.qkv, m->norm_out, m->qkv, MT, m->xs_scratch, st));
            nl += 3;
            IM_MARK(kCatQkv);
        } else {
            IM_TRY(im_cuda_residual_add(m->residual, m->ffn_down, m->hidden, (size_t)MT * H, st));
            nl++;
            IM_MARK(kCatResNorm);
        }
    }
    // Launch-per-kernel schedule with the reference's decode-time rounding points (one token per sequence):
    //   4-bit weights: Q of layers >= 1 comes out of the fused residual + norm + projection kernel (unrounded
    //   normalised vector), K and V read norm_out (metal/attention.rs:616-702); gate/up read norm_out and keep their
    //   f32 dot products for SiLU(g) * u (metal/ffn.rs:25-54).  Other widths have no fused kernels in the reference:
    //   every projection reads the fp16 buffers, gate and up are rounded before the activation (ffn.rs:58-150).
    for (int l = 0; l < c.num_layers && !mega && !gemm; l++) {
        Layer &L = m->layers[l];
        const bool fused4 = L.qkv->bits == 4 && L.gate->bits == 4 && L.up->bits == 4;
        const int nmv = (MT + 3) / 4;
        if (l == 0) {
            IM_TRY(im_cuda_matvec_affine(static_cast<const im_affine_weight *>(&L.q_rows), m->norm_out, m->q_d, MT, st));
            IM_TRY(im_cuda_matvec_affine(static_cast<const im_affine_weight *>(&L.kv_rows), m->norm_out, m->k_d, MT, st));
            nl += 2 * nmv;
            IM_MARK(kCatQkv);
        }
        // (QK-norm +) RoPE, K/V cache write and query rotation in one launch, then split attention + reduce
        TqPrep a{};
        a.qkv = m->q_d; a.stride = m->q_dim; a.kv = m->k_d; a.kv_stride = 2 * m->kv_dim; a.k_off = 0; a.v_off = m->kv_dim;
        a.qw = L.q_norm; a.kw = L.k_norm; a.cosc = m->cosc; a.sinc = m->sinc;
        a.nh = m->nh_l; a.nkv = m->nkv_l; a.rotary_dim = c.rotary_dim ? c.rotary_dim : hd; a.with_norm = c.qk_norm ? 1 : 0;
        a.T = T; a.nseq = nseq; a.max_seq = c.max_seq_len; a.base_pos = 0; a.eps = eps; a.pos_dev = m->pos_dev; a.slot_map = slots;
        a.qrot = m->qrot; a.q_out = nullptr;
        a.kc = L.kc; a.vc = L.vc; a.ks = L.ks; a.vs = L.vs; a.krn = L.krn;
        IM_TRY(attention_block(m, 0, a, m->q_d, L, nseq, T, attn_scale, attn_splits, slots, st));
        IM_MARK(kCatKvWrite);
        IM_TRY(attention_block(m, 1, a, m->q_d, L, nseq, T, attn_scale, attn_splits, slots, st));
        nl += 3;
        IM_MARK(kCatAttn);
        IM_TRY(im_cuda_matvec_affine(static_cast<im_affine_weight *>(L.o), m->attn_out, m->ffn_down, MT, st));
        IM_MARK(kCatOProj);
        IM_TRY(tp_allreduce(m, m->ffn_down, (size_t)MT * H, st));
        if (m->world > 1) IM_MARK(kCatComm);
        IM_TRY(im_cuda_fused_residual_rms_norm(m->hidden, m->ffn_down, L.post_ln, m->norm_out, m->residual, H, MT, eps, st));
        IM_MARK(kCatResNorm);
        if (fused4) {
            IM_TRY(im_cuda_ffn_gate_up_act(static_cast<im_affine_weight *>(L.gate), static_cast<im_affine_weight *>(L.up), m->norm_out,
                                           m->ffn_gate, MT, st));
            nl += nmv;
        } else {
            IM_TRY(im_cuda_matvec_affine(static_cast<im_affine_weight *>(L.gate), m->norm_out, m->ffn_gate, MT, st));
            IM_TRY(im_cuda_matvec_affine(static_cast<im_affine_weight *>(L.up), m->norm_out, m->ffn_up, MT, st));
            const size_t n = (size_t)MT * m->I_l;
            cudaError_t le = launch_k(silu_mul_kernel, dim3((unsigned)((n / 2 + 255) / 256)), dim3(256), 0, st, (const __half *)m->ffn_gate,
                                      (const __half *)m->ffn_up, m->ffn_gate, n);
            if (le != cudaSuccess) return fail(IM_ERR_CUDA, "launch failed: %s", cudaGetErrorString(le));
            nl += 2 * nmv + 1;
        }
        IM_MARK(kCatFfn);
        IM_TRY(im_cuda_matvec_affine(static_cast<im_affine_weight *>(L.down), m->ffn_gate, m->ffn_down, MT, st));
        IM_MARK(kCatDown);
        IM_TRY(tp_allreduce(m, m->ffn_down, (size_t)MT * H, st));
        if (m->world > 1) IM_MARK(kCatComm);
        nl += 2 * nmv + 1 + (m->world > 1 ? 2 : 0);
        if (l + 1 < c.num_layers) {
            Layer &Nx = m->layers[l + 1];
            if (Nx.qkv->bits == 4) {
                IM_TRY(im_cuda_fused_residual_norm_matvec(static_cast<const im_affine_weight *>(&Nx.q_rows), m->residual, m->ffn_down, Nx.input_ln,
                                                          eps, m->q_d, m->hidden, m->norm_out, MT, st));
            } else {
                IM_TRY(im_cuda_fused_residual_rms_norm(m->residual, m->ffn_down, Nx.input_ln, m->norm_out, m->hidden, H, MT, eps, st));
                IM_TRY(im_cuda_matvec_affine(static_cast<const im_affine_weight *>(&Nx.q_rows), m->norm_out, m->q_d, MT, st));
                nl++;
            }
            IM_TRY(im_cuda_matvec_affine(static_cast<const im_affine_weight *>(&Nx.kv_rows), m->norm_out, m->k_d, MT, st));
            nl += 2 * nmv;
            IM_MARK(kCatQkv);
        } else {
            IM_TRY(im_cuda_residual_add(m->residual, m->ffn_down, m->hidden, (size_t)MT * H, st));
            nl++;
            IM_MARK(kCatResNorm);
        }
    }
    if (all_logits) {  // final norm + lm_head on every token of the (single) sequence: prefill_all_logits
        IM_TRY(im_cuda_rms_norm(m->hidden, m->final_norm, m->norm_out, H, MT, eps, st));
        for (int r = 0; r < MT; r += 64) {  // the fp16 matvec takes up to 64 rows per call
            const int nb = MT - r < 64 ? MT - r : 64;
            IM_TRY(im_cuda_matvec_f16(m->lm_head, m->norm_out + (size_t)r * H, m->logits_seq + (size_t)r * m->vocab_l, m->vocab_l, H, nb, st));
        }
        nl += 1 + (MT + 3) / 4;
        if (m->world > 1) {
#if IM_HAVE_NCCL_H
            IM_NCCL_CHECK(nccl()->AllGather(m->logits_seq, m->logits_seq_all, (size_t)MT * m->vocab_l, ncclHalf, m->comm, st));
            nl++;
#endif
        }
        if (launches) *launches = nl;
        return IM_OK;
    }
    // final norm + lm_head on the last token of each sequence
    for (int s = 0; s < nseq; s++) {
        const __half *last = m->hidden + ((size_t)s * T + (T - 1)) * H;
        IM_TRY(im_cuda_rms_norm(last, m->final_norm, m->norm_out + (size_t)s * H, H, 1, eps, st));
        nl++;
    }
    IM_TRY(im_cuda_matvec_f16(m->lm_head, m->norm_out, m->logits, m->vocab_l, H, nseq, st));
    nl += (nseq + 3) / 4;
    if (m->world > 1) {
#if IM_HAVE_NCCL_H
        IM_NCCL_CHECK(nccl()->AllGather(m->logits, m->logits_all, (size_t)nseq * m->vocab_l, ncclHalf, m->comm, st));
        nl++;
#endif
    }
    IM_MARK(kCatHead);
    if (launches) *launches = nl;
    return IM_OK;
}

// Tables of the whole-token decode kernel.  Used when one sequence decodes on one GPU and every projection
// has the tiled INT4 layout; anything else keeps the launch-per-kernel schedule of forward().
static int mega_prepare(Model *m) {
    m->mega_ready = false;
    const im_model_config &c = m->cfg;
    if (c.decode_schedule == 1) return IM_OK;
    const bool tp = m->world > 1;
    // one GPU: opt-in only (measured slower there than the barrier: 64.0 against 60.0 us per layer at L8 shapes)
    const bool tagged = tp || c.decode_schedule == 2;
    if (c.tq_bits == 16) return IM_OK;           // fp16 cache: the per-kernel schedule
    if (tagged && c.tq_bits == 4) return IM_OK;  // 4-bit caches: the barrier form of the kernel only (tensor parallel: per-kernel schedule)
    if (tp && (!m->xar.ok || m->world > 8 || c.hidden_size % 128 != 0)) return IM_OK;  // needs the peer mapping of tp_init
    if (c.head_dim != 128 || m->nkv_l <= 0 || m->nh_l % m->nkv_l != 0) return IM_OK;
    const int gq = m->nh_l / m->nkv_l;
    if (gq != 1 && gq != 2 && gq != 4 && gq != 8) return IM_OK;
    int g_max = 0;
    for (Layer &L : m->layers) {
        for (AffineWeight *w : {L.qkv, L.o, L.gate, L.up, L.down}) {
            if (!w || !w->tiles || w->bits != 4 || w->group_size != 128) return IM_OK;
            if (w->G > g_max) g_max = w->G;
        }
        if (L.gate->N != L.up->N || L.gate->K != L.up->K) return IM_OK;
        if ((L.gate->awq != nullptr) != (L.up->awq != nullptr)) return IM_OK;
        IM_TRY(ensure_pair(L.gate, L.up, m->stream));
    }
    const int g_norm = c.hidden_size / 128;
    if (c.hidden_size % 128 != 0) return IM_OK;
    if (tagged && g_norm > 32) return IM_OK;  // the mailbox form of the norm staging keeps one chunk per thread (hidden <= 4096)
    const int u_bytes = mega_u_bytes(g_max, g_norm, gq);
    if (u_bytes < 0) return IM_OK;
    int nring = 8;
    while (nring >= 3 && mega_smem_bytes(nring, u_bytes) + 1024 > m->dev->smem_optin) nring--;
    if (nring < 3) return IM_OK;
    const int L = c.num_layers;
    std::vector<MegaPhase> ph((size_t)4 * L);
    std::vector<MegaLayer> ml((size_t)L);
    for (int l = 0; l < L; l++) {
        Layer &Ly = m->layers[l];
        MegaPhase q{}, o{}, gu{}, dn{};
        q.tiles = Ly.qkv->tiles; q.awq = Ly.qkv->awq; q.nblk = Ly.qkv->nblk; q.G = Ly.qkv->G; q.N = Ly.qkv->N; q.y = m->qkv;
        if (l == 0) {
            q.x = m->norm_out;
        } else {
            q.x = m->residual; q.resid = m->ffn_down; q.gamma = Ly.input_ln; q.resid_out = m->hidden;
            q.split_row = m->q_dim;  // Q from the unrounded vector, K and V from norm_out (metal/attention.rs:616-702)
        }
        o.tiles = Ly.o->tiles; o.awq = Ly.o->awq; o.nblk = Ly.o->nblk; o.G = Ly.o->G; o.N = Ly.o->N; o.x = m->attn_out; o.y = m->ffn_down;
        gu.tiles = Ly.gate->pair_tiles; gu.awq = Ly.gate->awq; gu.nblk = Ly.gate->pair_nblk; gu.G = Ly.gate->G; gu.N = Ly.gate->N;
        gu.x = m->hidden; gu.resid = m->ffn_down; gu.gamma = Ly.post_ln; gu.resid_out = m->residual; gu.y = m->ffn_gate; gu.gate_up = 1;
        dn.tiles = Ly.down->tiles; dn.awq = Ly.down->awq; dn.nblk = Ly.down->nblk; dn.G = Ly.down->G; dn.N = Ly.down->N;
        dn.x = m->ffn_gate; dn.y = m->ffn_down;
        if (tagged) {  // o and down hand their outputs over through the tagged mailboxes (tensor parallel: partial sums of
                       // the row-split projections, summed by the reader); no grid barrier follows them
            const int par = (l & 1) * 2;  // layers alternate between two pairs of mailboxes
            o.xout = 1 + par;
            gu.resid = m->ffn_down; gu.xin = 1 + par;        // resid stays non-null: it marks the norm phases
            if (l > 0) { q.resid = m->ffn_down; q.xin = 1 + ((l - 1) & 1) * 2 + 1; }
            if (l + 1 < L) dn.xout = 1 + par + 1;            // the last layer's output feeds the final norm outside the kernel
        }
        ph[4 * l] = q; ph[4 * l + 1] = o; ph[4 * l + 2] = gu; ph[4 * l + 3] = dn;
        ml[l] = MegaLayer{Ly.q_norm, Ly.k_norm, Ly.kc, Ly.vc, Ly.ks, Ly.vs, Ly.krn};
    }
    MegaParams &p = m->mega;
    p = MegaParams{};
    MegaPhase *dph = nullptr;
    MegaLayer *dml = nullptr;
    IM_TRY(m->alloc((void **)&dph, ph.size() * sizeof(MegaPhase)));
    IM_TRY(m->alloc((void **)&dml, ml.size() * sizeof(MegaLayer)));
    IM_CUDA_CHECK(cudaMemcpy(dph, ph.data(), ph.size() * sizeof(MegaPhase), cudaMemcpyHostToDevice));
    IM_CUDA_CHECK(cudaMemcpy(dml, ml.data(), ml.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice));
    p.phases = dph; p.layers = dml;
    p.L = L; p.nh = m->nh_l; p.nkv = m->nkv_l; p.q_dim = m->q_dim; p.kv_dim = m->kv_dim;
    p.pos = m->pos_dev; p.qkv = m->qkv; p.attn_out = m->attn_out; p.qrot = m->qrot;
    p.splits = m->dev->sm_count * 4 / m->nkv_l;
    if (p.splits < 1) p.splits = 1;
    if (p.splits > 256) p.splits = 256;
    const size_t rows = (size_t)m->nh_l * p.splits;
    float *part = nullptr;
    IM_TRY(m->alloc((void **)&part, rows * (128 + 2) * sizeof(float)));
    p.po = part; p.pm = part + rows * 128; p.pl = p.pm + rows;
    p.cosc = m->cosc; p.sinc = m->sinc;
    const Tq *tq = reinterpret_cast<const Tq *>(m->tq);
    p.signs = tq->signs; p.qjl_t = tq->qjl_t; p.k_cb = tq->k_cb; p.k_bd = tq->k_bd; p.v_cb = tq->v_cb; p.v_bd = tq->v_bd;
    p.k_levels = tq->k_levels; p.v_levels = tq->v_levels; p.tq_bits = tq->n_bits;
    p.eps = c.rms_eps;
    p.attn_scale = c.attn_scale != 0.0f ? c.attn_scale : 1.0f / sqrtf((float)c.head_dim);
    p.qjl_factor = sqrtf(2.0f / 3.14159265f) / (float)c.head_dim;
    p.max_seq = c.max_seq_len; p.rotary_dim = c.rotary_dim ? c.rotary_dim : c.head_dim; p.with_qk_norm = c.qk_norm ? 1 : 0;
    p.nring = nring; p.u_bytes = u_bytes; p.g_max = g_max; p.g_norm = g_norm; p.g_cap = mega_g_cap(g_max, g_norm);
    IM_TRY(m->alloc((void **)&p.bar, (size_t)(7 * L + 1) * sizeof(unsigned)));
    IM_CUDA_CHECK(cudaMemset(p.bar, 0, (size_t)(7 * L + 1) * sizeof(unsigned)));
    p.err = m->dev->err_flag;
    if (tp) {
        p.tagged = 1; p.world = m->world; p.rank = m->rank; p.xH = c.hidden_size;
        for (int r = 0; r < m->world; r++) p.xmail[r] = reinterpret_cast<uint2 *>(m->xar.peer[r] + m->xar.mail_off);
        p.xepoch = reinterpret_cast<unsigned *>(m->xar.base + m->xar.epoch_off);
    } else if (tagged) {  // one GPU: local mailboxes (4 x hidden/2 pairs per rank slot), then the launch count
        // sized for two rank slots: im_cuda_model_test_missing_ranks makes the kernel expect a second rank's sums
        const size_t mail_bytes = (size_t)4 * 2 * (c.hidden_size / 2) * sizeof(uint2);
        unsigned char *loc = nullptr, *phantom = nullptr;
        IM_TRY(m->alloc((void **)&loc, mail_bytes + 256));
        IM_TRY(m->alloc((void **)&phantom, mail_bytes));
        IM_CUDA_CHECK(cudaMemset(loc, 0, mail_bytes + 256));
        IM_CUDA_CHECK(cudaMemset(phantom, 0, mail_bytes));
        p.tagged = 1; p.world = 1; p.rank = 0; p.xH = c.hidden_size;
        p.xmail[0] = reinterpret_cast<uint2 *>(loc);
        p.xepoch = reinterpret_cast<unsigned *>(loc + mail_bytes);
        m->mega_capacity2 = true;
        m->mega_phantom_mail = reinterpret_cast<uint2 *>(phantom);
    }
    p.wait_ms = c.wait_limit_ms > 0 ? (unsigned)c.wait_limit_ms : 0u;
    // phase stamps of CTA 0 (a store per grid barrier; read back by im_cuda_model_token_kernel_profile)
    IM_TRY(m->alloc((void **)&p.trace, (size_t)(7 * L + 2) * sizeof(unsigned long long)));
    IM_CUDA_CHECK(cudaMemset(p.trace, 0, (size_t)(7 * L + 2) * sizeof(unsigned long long)));
    IM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
    m->mega_ready = true;
    return IM_OK;
}

static int decode_splits(const Model *m, int batch) {
    return tq_auto_splits(m->dev, batch, 1, m->nkv_l, m->cfg.max_seq_len);
}

// mapped: the sequences of the batch live in the slots listed in m->slot_map (continuous batching); otherwise in slots 0 .. batch - 1.
static int get_graph(Model *m, int batch, cudaGraphExec_t *out, bool mapped = false) {
    const int key = batch + (mapped ? 1000 : 0);
    const int *slots = mapped ? m->slot_map : nullptr;
    auto it = m->graphs.find(key);
    if (it != m->graphs.end()) {
        *out = it->second;
        return IM_OK;
    }
    cudaStream_t st = m->stream;
    // one eager pass first: sets function attributes and warms NCCL outside the capture
    const int splits = decode_splits(m, batch);
    IM_TRY(forward(m, batch, 1, splits, st, nullptr, nullptr, false, slots));
    IM_CUDA_CHECK(cudaStreamSynchronize(st));
    cudaGraph_t g = nullptr;
    IM_CUDA_CHECK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    int nl = 0;
    int rc = forward(m, batch, 1, splits, st, &nl, nullptr, false, slots);
    if (rc == IM_OK) {
        const __half *lg = m->world > 1 ? m->logits_all : m->logits;
        cudaError_t le = launch_k(argmax_kernel, dim3(kArgmaxCtas, batch), dim3(kArgmaxThreads), 0, st, lg, m->vocab_l, m->world, batch, m->tokens_dev,
                                  m->tok_hist, (const int *)m->step_dev, m->cfg.max_batch, m->cfg.max_seq_len, m->argmax_cand, m->argmax_counters);
        if (le == cudaSuccess) le = launch_k(bump_kernel, dim3(1), dim3(1), 0, st, m->step_dev);
        if (le == cudaSuccess) le = launch_k(advance_pos_kernel, dim3(1), dim3(64), 0, st, m->pos_dev, slots, batch, 1);
        if (le != cudaSuccess) rc = fail(IM_ERR_CUDA, "launch failed: %s", cudaGetErrorString(le));
        nl += 3;
    }
    cudaError_t e = cudaStreamEndCapture(st, &g);
    if (rc != IM_OK) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return fail(IM_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    cudaGraphExec_t ge = nullptr;
    e = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(IM_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
    m->graphs[key] = ge;
    m->launches_per_step = nl;
    *out = ge;
    return IM_OK;
}

// fp16 -> f32 on the host: 128 K logits per step.  With F16C (every x86-64-v3 CPU) eight at a time.
#if defined(__x86_64__)
__attribute__((target("avx,f16c"))) static void widen_f16c(const __half *src, float *dst, int n) {
    int j = 0;
    for (; j + 8 <= n; j += 8) _mm256_storeu_ps(dst + j, _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i *>(src + j))));
    for (; j < n; j++) dst[j] = __half2float(src[j]);
}
#endif
static void widen(const __half *src, float *dst, int n) {
#if defined(__x86_64__)
    static const bool have = __builtin_cpu_supports("f16c") && __builtin_cpu_supports("avx");
    if (have) return widen_f16c(src, dst, n);
#endif
    for (int j = 0; j < n; j++) dst[j] = __half2float(src[j]);
}
static void logits_to_host(const Model *m, const __half *pin, int nseq, float *out) {
    const int vl = m->vocab_l, parts = m->world, V = m->cfg.vocab_size;
    for (int p = 0; p < parts; p++)
        for (int s = 0; s < nseq; s++) widen(pin + ((size_t)p * nseq + s) * vl, out + (size_t)s * V + (size_t)p * vl, vl);
}

// A kernel whose bounded wait ran out leaves a non-zero word; the step's results are then invalid.  Clears the
// word and the grid-barrier counters so that the next step starts clean.
static int step_error_check(Model *m) {
    if (*m->err_pin == 0) return IM_OK;
    const int code = *m->err_pin;
    *m->err_pin = 0;
    cudaMemset(m->dev->err_flag, 0, sizeof(int));
    cudaMemset(m->dev->sk_counters, 0, (size_t)kSkMaxBlocks * sizeof(int));
    if (m->mega.bar) cudaMemset(m->mega.bar, 0, (size_t)(7 * m->cfg.num_layers + 1) * sizeof(unsigned));
    return fail(IM_ERR_TIMEOUT, "a device-side bounded wait ran out (code %d); the results of this step are invalid", code);
}

// Positions of every slot (reset, truncate of the single-sequence / lockstep interface).
static int set_positions(Model *m, int pos) {
    set_pos_kernel<<<1, 64, 0, m->stream>>>(m->pos_dev, m->cfg.max_batch, pos);
    IM_CUDA_CHECK(cudaGetLastError());
    for (int &p : m->slot_pos) p = pos;
    return IM_OK;
}
__global__ void set_one_pos_kernel(int *pos, int slot, int v) { pos[slot] = v; }

// Prefill of n tokens into cache slot `slot`, continuing at that slot's position.  last_logits (optional): f32 [vocab]
// of the last token; all_logits (optional): f32 [n, vocab].
static int prefill_slot(Model *m, int slot, const uint32_t *tokens_host, int n, float *last_logits, float *all_logits) {
    if (m->slot_pos[slot] + n > m->cfg.max_seq_len)
        return fail(IM_ERR_BOUNDS, "sequence position %d + %d tokens exceeds max_seq_len %d", m->slot_pos[slot], n, m->cfg.max_seq_len);
    cudaStream_t st = m->stream;
    // 256-token chunks when the projections run as tensor-core GEMMs; the matvec kernels take at most 64 rows per call
    int chunk = m->gemm_ok ? m->cfg.prefill_chunk_size : (m->cfg.prefill_chunk_size < 64 ? m->cfg.prefill_chunk_size : 64);
    if (all_logits && chunk > kAllLogitsChunk) chunk = kAllLogitsChunk;
    const size_t V = (size_t)m->cfg.vocab_size;
    const int *slots = slot == 0 ? nullptr : m->slot_ident + slot;
    if (all_logits && !m->logits_seq) {  // first use: a chunk's worth of logits on the device and in pinned host memory
        IM_TRY(m->alloc((void **)&m->logits_seq, (size_t)kAllLogitsChunk * m->vocab_l * 2));
        if (m->world > 1) IM_TRY(m->alloc((void **)&m->logits_seq_all, (size_t)kAllLogitsChunk * V * 2));
        IM_CUDA_CHECK(cudaMallocHost((void **)&m->logits_seq_pin, (size_t)kAllLogitsChunk * V * 2));
    }
    for (int done = 0; done < n; done += chunk) {
        const int T = n - done < chunk ? n - done : chunk;
        memcpy(m->tokens_pin, tokens_host + done, (size_t)T * 4);
        IM_CUDA_CHECK(cudaMemcpyAsync(m->tokens_dev, m->tokens_pin, (size_t)T * 4, cudaMemcpyHostToDevice, st));
        const int splits = tq_auto_splits(m->dev, 1, T, m->nkv_l, m->slot_pos[slot] + T);
        m->prefill_slot_id = slot;
        m->prefill_ctx_end = m->slot_pos[slot] + T;
        const int frc = forward(m, 1, T, splits, st, nullptr, nullptr, all_logits != nullptr, slots);
        m->prefill_slot_id = -1;
        IM_TRY(frc);
        advance_pos_kernel<<<1, 64, 0, st>>>(m->pos_dev, slots, 1, T);
        IM_CUDA_CHECK(cudaGetLastError());
        if (all_logits) {
            const __half *lg = m->world > 1 ? m->logits_seq_all : m->logits_seq;
            IM_CUDA_CHECK(cudaMemcpyAsync(m->logits_seq_pin, lg, (size_t)T * V * 2, cudaMemcpyDeviceToHost, st));
        }
        IM_CUDA_CHECK(cudaMemcpyAsync(m->err_pin, m->dev->err_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
        IM_CUDA_CHECK(cudaStreamSynchronize(st));  // tokens_pin is reused by the next chunk
        IM_TRY(step_error_check(m));
        m->slot_pos[slot] += T;
        if (all_logits) {  // device layout [part][token][vocab_l] -> host rows [token][vocab]
            const int vl = m->vocab_l;
            for (int p = 0; p < m->world; p++)
                for (int t = 0; t < T; t++)
                    widen(m->logits_seq_pin + ((size_t)p * T + t) * vl, all_logits + (size_t)(done + t) * V + (size_t)p * vl, vl);
        }
    }
    if (last_logits) {
        const __half *lg = m->world > 1 ? m->logits_all : m->logits;
        IM_CUDA_CHECK(cudaMemcpyAsync(m->logits_pin, lg, V * 2, cudaMemcpyDeviceToHost, st));
        IM_CUDA_CHECK(cudaStreamSynchronize(st));
        logits_to_host(m, m->logits_pin, 1, last_logits);
    }
    return IM_OK;
}

}  // namespace im

using namespace im;
struct im_model : im::Model {};

IM_EXPORT int im_cuda_tp_unique_id(void *id_out_128_bytes) {
    IM_GUARD_BEGIN
    IM_REQUIRE(id_out_128_bytes, "bad argument");
#if IM_HAVE_NCCL_H
    if (!nccl()) return fail(IM_ERR_NCCL, "libnccl.so.2 could not be loaded");
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    ncclUniqueId id;
    IM_NCCL_CHECK(nccl()->GetUniqueId(&id));
    memcpy(id_out_128_bytes, &id, 128);
    return IM_OK;
#else
    return fail(IM_ERR_NCCL, "built without nccl.h");
#endif
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_tp_init(im_model *m, const void *id_128_bytes) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && id_128_bytes, "bad argument");
    if (m->world <= 1) return IM_OK;
#if IM_HAVE_NCCL_H
    if (!nccl()) return fail(IM_ERR_NCCL, "libnccl.so.2 could not be loaded");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    ncclUniqueId id;
    memcpy(&id, id_128_bytes, 128);
    IM_NCCL_CHECK(nccl()->CommInitRank(&m->comm, m->world, id, m->rank));
    // Receive buffers of the one-shot all-reduce, mapped into every rank with CUDA IPC (handles exchanged through the
    // communicator just created).  Any failure here leaves the NCCL all-reduce in charge.
    if (m->world <= kXarMaxWorld && m->cfg.tp_collective != 1) {
        PeerAllreduce &x = m->xar;
        x.cap = (size_t)4 * m->cfg.hidden_size;  // up to four batch rows: the decode batches that run one matvec per projection
        x.bytes = 256 + (size_t)2 * m->world * x.cap * sizeof(__half);
        x.mail_off = (x.bytes + 255) & ~(size_t)255;
        x.epoch_off = (x.mail_off + (size_t)4 * m->world * (m->cfg.hidden_size / 2) * sizeof(uint2) + 255) & ~(size_t)255;
        x.bytes = x.epoch_off + 256;
        cudaIpcMemHandle_t mine{};
        unsigned char *xchg = nullptr;
        std::vector<cudaIpcMemHandle_t> all((size_t)m->world);
        bool good = cudaMalloc((void **)&x.base, x.bytes) == cudaSuccess && cudaMemset(x.base, 0, x.bytes) == cudaSuccess &&
                    cudaIpcGetMemHandle(&mine, x.base) == cudaSuccess &&
                    cudaMalloc((void **)&xchg, (size_t)m->world * sizeof(mine)) == cudaSuccess &&
                    cudaMemcpy(xchg + (size_t)m->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice) == cudaSuccess;
        // every rank takes part in the exchange whatever happened locally (a rank that failed sends zeros)
        ncclResult_t nr = nccl()->AllGather(xchg ? xchg + (size_t)m->rank * sizeof(mine) : nullptr, xchg, sizeof(mine), ncclChar, m->comm,
                                            m->stream);
        good = good && nr == ncclSuccess && cudaStreamSynchronize(m->stream) == cudaSuccess &&
               cudaMemcpy(all.data(), xchg, (size_t)m->world * sizeof(mine), cudaMemcpyDeviceToHost) == cudaSuccess;
        for (int p = 0; good && p < m->world; p++) {
            if (p == m->rank) {
                x.peer[p] = x.base;
                continue;
            }
            void *ptr = nullptr;
            good = cudaIpcOpenMemHandle(&ptr, all[(size_t)p], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
            x.peer[p] = static_cast<unsigned char *>(ptr);
        }
        if (xchg) cudaFree(xchg);
        (void)cudaGetLastError();
        // all ranks must agree: one that could not map its peers would wait for flags nobody raises
        int *agree = nullptr;
        int flag = good ? 1 : 0, out = 0;
        if (cudaMalloc((void **)&agree, sizeof(int)) == cudaSuccess) {
            cudaMemcpy(agree, &flag, sizeof(int), cudaMemcpyHostToDevice);
            if (nccl()->AllReduce(agree, agree, 1, ncclInt, ncclMin, m->comm, m->stream) == ncclSuccess &&
                cudaStreamSynchronize(m->stream) == cudaSuccess)
                cudaMemcpy(&out, agree, sizeof(int), cudaMemcpyDeviceToHost);
            cudaFree(agree);
        }
        x.ok = out == 1;
        (void)cudaGetLastError();
        // Known-answer check of the mapping before anything depends on it: rank r contributes r + 1 in every element,
        // three calls (both buffer parities, then the first again); every rank must read world (world + 1) / 2 everywhere.
        // Any rank that does not sends everybody back to NCCL.
        if (x.ok) {
            const size_t n = (size_t)m->cfg.hidden_size;
            std::vector<__half> hv(n, __float2half((float)(m->rank + 1)));
            __half *tv = nullptr;
            int good_kat = cudaMalloc((void **)&tv, n * sizeof(__half)) == cudaSuccess ? 1 : 0;
            const float want = 0.5f * (float)m->world * (float)(m->world + 1);
            for (int it = 0; it < 3; it++) {  // every rank launches all three, whatever it has seen so far
                if (tv) cudaMemcpyAsync(tv, hv.data(), n * sizeof(__half), cudaMemcpyHostToDevice, m->stream);
                if (tv && n <= x.cap && n % 8 == 0) {
                    if (tp_allreduce(m, tv, n, m->stream) != IM_OK) good_kat = 0;
                } else {
                    good_kat = 0;
                }
                std::vector<__half> back(n);
                if (!tv || cudaMemcpyAsync(back.data(), tv, n * sizeof(__half), cudaMemcpyDeviceToHost, m->stream) != cudaSuccess ||
                    cudaStreamSynchronize(m->stream) != cudaSuccess)
                    good_kat = 0;
                for (size_t i = 0; good_kat && i < n; i++)
                    if (__half2float(back[i]) != want) good_kat = 0;
            }
            int errw = 0;
            cudaMemcpy(&errw, m->dev->err_flag, sizeof(int), cudaMemcpyDeviceToHost);
            if (errw != 0) {
                good_kat = 0;
                cudaMemset(m->dev->err_flag, 0, sizeof(int));
            }
            if (tv) cudaFree(tv);
            int all_kat = 0;
            int *ag = nullptr;
            if (cudaMalloc((void **)&ag, sizeof(int)) == cudaSuccess) {
                cudaMemcpy(ag, &good_kat, sizeof(int), cudaMemcpyHostToDevice);
                if (nccl()->AllReduce(ag, ag, 1, ncclInt, ncclMin, m->comm, m->stream) == ncclSuccess &&
                    cudaStreamSynchronize(m->stream) == cudaSuccess)
                    cudaMemcpy(&all_kat, ag, sizeof(int), cudaMemcpyDeviceToHost);
                cudaFree(ag);
            }
            x.ok = all_kat == 1;
            (void)cudaGetLastError();
        }
        // The whole-token kernel exchanges its row-split partial sums through the same mapping; every rank must run it
        // or none (a rank on the per-kernel schedule would never feed the others' counters).
        if (x.ok) {
            int mine_ready = 0;
            if (mega_prepare(m) == IM_OK && m->mega_ready) mine_ready = 1;
            int all_ready = 0;
            int *ag = nullptr;
            if (cudaMalloc((void **)&ag, sizeof(int)) == cudaSuccess) {
                cudaMemcpy(ag, &mine_ready, sizeof(int), cudaMemcpyHostToDevice);
                if (nccl()->AllReduce(ag, ag, 1, ncclInt, ncclMin, m->comm, m->stream) == ncclSuccess &&
                    cudaStreamSynchronize(m->stream) == cudaSuccess)
                    cudaMemcpy(&all_ready, ag, sizeof(int), cudaMemcpyDeviceToHost);
                cudaFree(ag);
            }
            if (all_ready != 1) m->mega_ready = false;
            (void)cudaGetLastError();
        }
    }
    return IM_OK;
#else
    return fail(IM_ERR_NCCL, "built without nccl.h");
#endif
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_create(im_device *dev, const im_model_config *cfg, im_model **out) {
    IM_GUARD_BEGIN
    IM_REQUIRE(dev && cfg && out, "bad argument");
    *out = nullptr;
    im_model_config c = *cfg;
    if (c.max_seq_len == 0) c.max_seq_len = 2048;
    if (c.max_batch == 0) c.max_batch = 1;
    if (c.tq_bits == 0) c.tq_bits = 8;
    if (c.rotation_seed == 0) c.rotation_seed = 42;
    if (c.tp_world == 0) c.tp_world = 1;
    // MetalConfig::validate (crates/ironmill-inference/src/metal/config.rs:364-384)
    IM_REQUIRE(c.max_seq_len > 0, "max_seq_len must be > 0");
    IM_REQUIRE(c.tq_bits == 4 || c.tq_bits == 8 || c.tq_bits == 16, "n_bits must be 4 or 8 (TurboQuant) or 16 (fp16 KV cache, TurboQuant off), got %d",
               c.tq_bits);
    IM_REQUIRE(c.num_layers > 0 && c.hidden_size > 0 && c.intermediate_size > 0 && c.num_heads > 0 && c.num_kv_heads > 0 &&
                   c.head_dim > 0 && c.vocab_size > 0, "model dimensions must be positive");
    IM_REQUIRE(c.head_dim == 128, "head_dim %d is not built (128 only)", c.head_dim);
    IM_REQUIRE(c.num_heads % c.num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads");
    IM_REQUIRE(c.max_batch >= 1 && c.max_batch <= 64, "max_batch must be in 1..64");
    IM_REQUIRE(c.tp_world >= 1 && c.tp_rank >= 0 && c.tp_rank < c.tp_world, "bad tensor-parallel rank %d of %d", c.tp_rank, c.tp_world);
    IM_REQUIRE(c.num_kv_heads % c.tp_world == 0 && c.intermediate_size % (c.tp_world * 128) == 0 && c.vocab_size % c.tp_world == 0,
               "tensor-parallel size %d must divide num_kv_heads, intermediate_size/128 and vocab_size", c.tp_world);
    IM_REQUIRE(c.rms_eps > 0.0f && c.rope_theta > 0.0, "rms_eps and rope_theta must be positive");
    IM_REQUIRE(c.prefill_chunk_size >= 0 && c.prefill_chunk_size <= kPrefillChunk, "prefill_chunk_size must be in 0..%d", kPrefillChunk);
    IM_REQUIRE(c.decode_schedule >= 0 && c.decode_schedule <= 2 && c.tp_collective >= 0 && c.tp_collective <= 1 && c.wait_limit_ms >= 0,
               "bad decode_schedule / tp_collective / wait_limit_ms");
    if (c.prefill_chunk_size == 0) c.prefill_chunk_size = kPrefillChunk;
    if (c.prefill_chunk_size > c.max_seq_len) c.prefill_chunk_size = c.max_seq_len;  // no prompt is longer than the cache
    IM_CUDA_CHECK(cudaSetDevice(dev->ordinal));
    im_model *m = new im_model();
    m->dev = dev;
    m->cfg = c;
    m->world = c.tp_world;
    m->rank = c.tp_rank;
    m->nh_l = c.num_heads / m->world;
    m->nkv_l = c.num_kv_heads / m->world;
    m->I_l = c.intermediate_size / m->world;
    m->vocab_l = c.vocab_size / m->world;
    m->q_dim = m->nh_l * c.head_dim;
    m->kv_dim = m->nkv_l * c.head_dim;
    m->qkv_dim = m->q_dim + 2 * m->kv_dim;
    m->layers.resize(c.num_layers);
    cudaError_t e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete m;
        return fail(IM_ERR_CUDA, "stream creation failed: %s", cudaGetErrorString(e));
    }
    *out = m;
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT void im_cuda_model_free(im_model *m) {
    if (!m) return;
    cudaSetDevice(m->dev->ordinal);
    if (m->stream) cudaStreamSynchronize(m->stream);
    for (auto &g : m->graphs) cudaGraphExecDestroy(g.second);
#if IM_HAVE_NCCL_H
    for (int p = 0; p < kXarMaxWorld; p++)
        if (m->xar.peer[p] && p != m->rank) cudaIpcCloseMemHandle(m->xar.peer[p]);
    if (m->xar.base) cudaFree(m->xar.base);
    if (m->comm && nccl() && nccl()->CommDestroy) nccl()->CommDestroy(m->comm);
#endif
    for (auto &L : m->layers) {
        im_cuda_affine_weight_free(static_cast<im_affine_weight *>(L.qkv));
        im_cuda_affine_weight_free(static_cast<im_affine_weight *>(L.o));
        im_cuda_affine_weight_free(static_cast<im_affine_weight *>(L.gate));
        im_cuda_affine_weight_free(static_cast<im_affine_weight *>(L.up));
        im_cuda_affine_weight_free(static_cast<im_affine_weight *>(L.down));
    }
    if (m->tq) im_cuda_tq_free(m->tq);
    for (auto &a : m->allocs) dev_free(m->dev, a.first, a.second);
    if (m->tokens_pin) cudaFreeHost(m->tokens_pin);
    if (m->logits_pin) cudaFreeHost(m->logits_pin);
    if (m->logits_seq_pin) cudaFreeHost(m->logits_seq_pin);
    if (m->slot_pin) cudaFreeHost(m->slot_pin);
    if (m->err_pin) cudaFreeHost(m->err_pin);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
}

IM_EXPORT int im_cuda_model_load_dense(im_model *m, const char *name, const void *data_f16_host, size_t n) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && name && data_f16_host, "bad argument");
    if (m->finalized) return fail(IM_ERR_STATE, "model already finalized");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    const im_model_config &c = m->cfg;
    const size_t H = c.hidden_size;
    std::string nm(name), suffix;
    int l = -1;
    if (nm == "model.embed_tokens.weight") {
        IM_REQUIRE(n == (size_t)c.vocab_size * H, "%s: expected %zu elements, got %zu", name, (size_t)c.vocab_size * H, n);
        return upload_f16(m, &m->embed, data_f16_host, n);
    }
    if (nm == "model.norm.weight") {
        IM_REQUIRE(n == H, "%s: expected %zu elements, got %zu", name, H, n);
        return upload_f16(m, &m->final_norm, data_f16_host, n);
    }
    if (nm == "lm_head.weight") {
        IM_REQUIRE(n == (size_t)c.vocab_size * H, "%s: expected %zu elements, got %zu", name, (size_t)c.vocab_size * H, n);
        const __half *src = static_cast<const __half *>(data_f16_host) + (size_t)m->rank * m->vocab_l * H;
        m->lm_head_owned = true;
        return upload_f16(m, &m->lm_head, src, (size_t)m->vocab_l * H);
    }
    if (parse_layer_name(name, &l, &suffix)) {
        IM_REQUIRE(l >= 0 && l < c.num_layers, "%s: layer index out of range", name);
        Layer &L = m->layers[l];
        if (suffix == "input_layernorm.weight") { IM_REQUIRE(n == H, "%s: bad size", name); return upload_f16(m, &L.input_ln, data_f16_host, n); }
        if (suffix == "post_attention_layernorm.weight") { IM_REQUIRE(n == H, "%s: bad size", name); return upload_f16(m, &L.post_ln, data_f16_host, n); }
        if (suffix == "self_attn.q_norm.weight") { IM_REQUIRE(n == (size_t)c.head_dim, "%s: bad size", name); return upload_f16(m, &L.q_norm, data_f16_host, n); }
        if (suffix == "self_attn.k_norm.weight") { IM_REQUIRE(n == (size_t)c.head_dim, "%s: bad size", name); return upload_f16(m, &L.k_norm, data_f16_host, n); }
    }
    return fail(IM_ERR_INVALID, "unknown dense tensor '%s'", name);
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_load_affine(im_model *m, const char *name, const void *qdata_host, const void *scales_host,
                                        const void *zeros_host, int param_dtype, const void *awq_f16_host, int N, int K,
                                        int group_size, int bit_width) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && name && qdata_host && scales_host && zeros_host, "bad argument");
    if (m->finalized) return fail(IM_ERR_STATE, "model already finalized");
    IM_REQUIRE(bit_width == 4 || bit_width == 8, "bit_width must be 4 or 8");
    IM_REQUIRE(group_size > 0, "group_size must be positive");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    const im_model_config &c = m->cfg;
    const int H = c.hidden_size, hd = c.head_dim, r = m->rank;
    std::string suffix;
    int l = -1;
    if (std::string(name) == "model.embed_tokens.weight" || std::string(name) == "lm_head.weight") {
        // An affine-quantized embedding table or lm_head (the reference accepts both,
        // crates/ironmill-inference/src/metal/weights.rs:305-420): dequantised here to the dense fp16 form the gather
        // and the lm_head matvec read: f16((q - z) * s) from the fp16 parameters the GPU kernels see
        // (crates/ironmill-core/src/dequant.rs:85-180,305-345), divided by the AWQ scale of its column if there is one.
        IM_REQUIRE(N == c.vocab_size && K == H, "%s: expected shape [%d,%d], got [%d,%d]", name, c.vocab_size, H, N, K);
        const int G = (K + group_size - 1) / group_size;
        std::vector<__half> dense((size_t)N * K);
        const uint8_t *q = static_cast<const uint8_t *>(qdata_host);
        auto param = [&](const void *p, size_t i) -> float {
            const float v = param_dtype == IM_DTYPE_F32 ? static_cast<const float *>(p)[i] : __half2float(static_cast<const __half *>(p)[i]);
            return __half2float(__float2half_rn(v));
        };
        const __half *awq = static_cast<const __half *>(awq_f16_host);
        for (size_t n = 0; n < (size_t)N; n++)
            for (int k = 0; k < K; k++) {
                const size_t e = n * K + k, pi = n * G + k / group_size;
                const unsigned code = bit_width == 4 ? (q[e >> 1] >> (4 * (e & 1))) & 15u : q[e];
                float v = __half2float(__float2half_rn(((float)code - param(zeros_host, pi)) * param(scales_host, pi)));
                if (awq) v = v / __half2float(awq[k]);
                dense[e] = __float2half_rn(v);
            }
        return im_cuda_model_load_dense(m, name, dense.data(), dense.size());
    }
    if (!parse_layer_name(name, &l, &suffix) || l < 0 || l >= c.num_layers) return fail(IM_ERR_INVALID, "unknown quantized tensor '%s'", name);
    Layer &L = m->layers[l];
    HostAffine h;
    auto expect = [&](int en, int ek) -> int {
        if (N != en || K != ek) return fail(IM_ERR_INVALID, "%s: expected shape [%d,%d], got [%d,%d]", name, en, ek, N, K);
        return IM_OK;
    };
    int r0, nr, c0, nc, en, ek;
    if (shard_rect(c, suffix, &r0, &nr, &c0, &nc, &en, &ek) != IM_OK) return fail(IM_ERR_INVALID, "unknown quantized tensor '%s'", name);
    IM_TRY(expect(en, ek));
    IM_TRY(slice_affine(&h, qdata_host, scales_host, zeros_host, param_dtype, awq_f16_host, N, K, group_size, bit_width, r0, nr, c0, nc));
    (void)H; (void)hd; (void)r;
    if (suffix == "self_attn.q_proj.weight") { L.hq = std::move(h); return IM_OK; }
    if (suffix == "self_attn.k_proj.weight") { L.hk = std::move(h); return IM_OK; }
    if (suffix == "self_attn.v_proj.weight") { L.hv = std::move(h); return IM_OK; }
    AffineWeight **dst = suffix == "self_attn.o_proj.weight" ? &L.o : suffix == "mlp.gate_proj.weight" ? &L.gate
                         : suffix == "mlp.up_proj.weight" ? &L.up : &L.down;
    if (*dst) return fail(IM_ERR_STATE, "%s loaded twice", name);
    return make_weight(m, h, dst);
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_set_tq_constants(im_model *m, const float *signs_host, const float *qjl_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && signs_host && qjl_host, "bad argument");
    if (m->finalized) return fail(IM_ERR_STATE, "model already finalized");
    const size_t hd = m->cfg.head_dim;
    m->signs_host.assign(signs_host, signs_host + hd);
    m->qjl_host.assign(qjl_host, qjl_host + hd * hd);
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_finalize(im_model *m) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m, "bad argument");
    if (m->finalized) return IM_OK;
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    const im_model_config &c = m->cfg;
    const int H = c.hidden_size, hd = c.head_dim;
    if (!m->embed) return fail(IM_ERR_STATE, "missing tensor model.embed_tokens.weight");
    if (!m->final_norm) return fail(IM_ERR_STATE, "missing tensor model.norm.weight");
    if (!m->lm_head) {
        if (!c.tie_word_embeddings) return fail(IM_ERR_STATE, "missing tensor lm_head.weight (and tie_word_embeddings is off)");
        m->lm_head = m->embed + (size_t)m->rank * m->vocab_l * H;  // tied: this rank's rows of the embedding table
    }
    for (int l = 0; l < c.num_layers; l++) {
        Layer &L = m->layers[l];
        if (!L.hq.have || !L.hk.have || !L.hv.have || !L.o || !L.gate || !L.up || !L.down || !L.input_ln || !L.post_ln)
            return fail(IM_ERR_STATE, "layer %d is missing tensors", l);
        if (c.qk_norm && (!L.q_norm || !L.k_norm)) return fail(IM_ERR_STATE, "layer %d is missing q_norm / k_norm", l);
        // concatenate q | k | v rows: they read the same input, so one launch serves all three
        const HostAffine &q = L.hq, &k = L.hk, &v = L.hv;
        if (q.K != k.K || q.K != v.K || q.gs != k.gs || q.gs != v.gs || q.bits != k.bits || q.bits != v.bits ||
            q.param_f32 != k.param_f32 || q.param_f32 != v.param_f32 || q.awq != k.awq || q.awq != v.awq)
            return fail(IM_ERR_INVALID, "layer %d: q/k/v projections must share K, group size, bit width, parameter dtype and AWQ scales", l);
        HostAffine f;
        f.N = q.N + k.N + v.N; f.K = q.K; f.gs = q.gs; f.bits = q.bits; f.param_f32 = q.param_f32; f.have = true; f.awq = q.awq;
        for (const HostAffine *p : {&q, &k, &v}) {
            f.q.insert(f.q.end(), p->q.begin(), p->q.end());
            f.s.insert(f.s.end(), p->s.begin(), p->s.end());
            f.z.insert(f.z.end(), p->z.begin(), p->z.end());
            f.s16.insert(f.s16.end(), p->s16.begin(), p->s16.end());
            f.z16.insert(f.z16.end(), p->z16.begin(), p->z16.end());
        }
        IM_TRY(make_weight(m, f, &L.qkv));
        L.q_rows = row_view(L.qkv, 0, m->q_dim);
        L.kv_rows = row_view(L.qkv, m->q_dim, 2 * m->kv_dim);
        L.hq = HostAffine(); L.hk = HostAffine(); L.hv = HostAffine();
        // KV cache of this rank's heads (MetalKvCache, crates/ironmill-inference/src/metal/turboquant/cache.rs:104-354)
        const size_t rows = (size_t)c.max_batch * m->nkv_l * c.max_seq_len;
        const size_t rowb = (size_t)hd * c.tq_bits / 8;  // one byte per element, or two elements per byte (n_bits = 4)
        IM_TRY(m->alloc((void **)&L.kc, rows * rowb));
        IM_TRY(m->alloc((void **)&L.vc, rows * rowb));
        IM_TRY(m->alloc((void **)&L.ks, rows * 4));
        IM_TRY(m->alloc((void **)&L.vs, rows * 4));
        IM_TRY(m->alloc((void **)&L.krn, rows * 4));
        IM_CUDA_CHECK(cudaMemset(L.ks, 0, rows * 4));
        IM_CUDA_CHECK(cudaMemset(L.vs, 0, rows * 4));
        IM_CUDA_CHECK(cudaMemset(L.krn, 0, rows * 4));
        IM_CUDA_CHECK(cudaMemset(L.kc, 0, rows * rowb));
        IM_CUDA_CHECK(cudaMemset(L.vc, 0, rows * rowb));
    }
    // TurboQuant constants
    if (m->signs_host.empty()) {
        m->signs_host.resize(hd);
        m->qjl_host.resize((size_t)hd * hd);
        IM_TRY(im_cuda_tq_generate(hd, c.rotation_seed, m->signs_host.data(), m->qjl_host.data()));
    }
    // (an fp16 cache keeps the handle for its scratch bookkeeping only: none of its tables is read)
    IM_TRY(im_cuda_tq_create(static_cast<im_device *>(m->dev), hd, c.tq_bits == 16 ? 8 : c.tq_bits, m->signs_host.data(), m->qjl_host.data(), nullptr,
                             nullptr, nullptr, nullptr, &m->tq));
    // RoPE tables
    IM_TRY(m->alloc((void **)&m->cosc, (size_t)c.max_seq_len * (hd / 2) * 2));
    IM_TRY(m->alloc((void **)&m->sinc, (size_t)c.max_seq_len * (hd / 2) * 2));
    IM_TRY(im_cuda_rope_table(hd, c.max_seq_len, c.rope_theta, c.rotary_dim, m->cosc, m->sinc));
    // activations
    m->MT = std::max(std::max(c.max_batch, c.prefill_chunk_size), kAllLogitsChunk < c.max_seq_len ? kAllLogitsChunk : c.max_seq_len);
    const size_t MT = m->MT;
    IM_TRY(m->alloc((void **)&m->hidden, MT * H * 2));
    IM_TRY(m->alloc((void **)&m->norm_out, MT * H * 2));
    IM_TRY(m->alloc((void **)&m->residual, MT * H * 2));
    IM_TRY(m->alloc((void **)&m->qkv, MT * m->qkv_dim * 2));
    IM_TRY(m->alloc((void **)&m->q_d, MT * m->q_dim * 2));
    IM_TRY(m->alloc((void **)&m->k_d, MT * 2 * m->kv_dim * 2));  // K | V rows of a token (launch-per-kernel schedule)
    IM_TRY(m->alloc((void **)&m->attn_out, MT * m->q_dim * 2));
    IM_TRY(m->alloc((void **)&m->qrot, MT * m->q_dim * 2 * sizeof(float)));
    IM_TRY(m->alloc((void **)&m->ffn_down, MT * H * 2));
    IM_TRY(m->alloc((void **)&m->ffn_gate, MT * m->I_l * 2));
    IM_TRY(m->alloc((void **)&m->ffn_up, MT * m->I_l * 2));
    {
        size_t kmax = (size_t)H;
        if ((size_t)m->I_l > kmax) kmax = (size_t)m->I_l;
        if ((size_t)m->q_dim > kmax) kmax = (size_t)m->q_dim;
        IM_TRY(m->alloc((void **)&m->xs_scratch, MT * kmax * 2));
    }
    m->gemm_ok = true;
    for (Layer &L : m->layers)
        for (AffineWeight *w : {L.qkv, L.o, L.gate, L.up, L.down})
            if (!w || (w->bits != 4 && w->bits != 8) || w->group_size != 128 || w->K % 128 != 0 || w->N % 8 != 0) m->gemm_ok = false;
    IM_TRY(m->alloc((void **)&m->logits, (size_t)c.max_batch * m->vocab_l * 2));
    if (m->world > 1) IM_TRY(m->alloc((void **)&m->logits_all, (size_t)c.max_batch * c.vocab_size * 2));
    IM_TRY(m->alloc((void **)&m->tokens_dev, MT * 4));
    IM_TRY(m->alloc((void **)&m->tok_hist, (size_t)c.max_seq_len * c.max_batch * 4));
    IM_TRY(m->alloc((void **)&m->pos_dev, 64 * 4));
    IM_TRY(m->alloc((void **)&m->slot_ident, 64 * 4));
    IM_TRY(m->alloc((void **)&m->slot_map, 64 * 4));
    {
        int ident[64];
        for (int i = 0; i < 64; i++) ident[i] = i;
        IM_CUDA_CHECK(cudaMemcpy(m->slot_ident, ident, sizeof(ident), cudaMemcpyHostToDevice));
        IM_CUDA_CHECK(cudaMemcpy(m->slot_map, ident, sizeof(ident), cudaMemcpyHostToDevice));
    }
    IM_CUDA_CHECK(cudaMallocHost((void **)&m->slot_pin, 64 * sizeof(int)));
    m->slot_pos.assign((size_t)c.max_batch, 0);
    m->slot_used.assign((size_t)c.max_batch, 0);
    IM_TRY(m->alloc((void **)&m->step_dev, 4));
    IM_CUDA_CHECK(cudaMemset(m->pos_dev, 0, 64 * 4));
    IM_CUDA_CHECK(cudaMemset(m->step_dev, 0, 4));
    IM_TRY(m->alloc((void **)&m->argmax_cand, (size_t)c.max_batch * kArgmaxCtas * sizeof(float2)));
    IM_TRY(m->alloc((void **)&m->argmax_counters, (size_t)c.max_batch * sizeof(unsigned)));
    IM_CUDA_CHECK(cudaMemset(m->argmax_counters, 0, (size_t)c.max_batch * sizeof(unsigned)));
    IM_CUDA_CHECK(cudaMallocHost((void **)&m->tokens_pin, MT * 4));
    IM_CUDA_CHECK(cudaMallocHost((void **)&m->logits_pin, (size_t)c.max_batch * c.vocab_size * 2));
    IM_CUDA_CHECK(cudaMallocHost((void **)&m->err_pin, sizeof(int)));
    *m->err_pin = 0;
    // attention scratch for the largest launch: decode at max_batch, or a prefill chunk
    size_t need = 0;
    for (int b = 1; b <= c.max_batch; b++) {
        const size_t s = im_cuda_tq_scratch_bytes(b, 1, m->nh_l, hd, decode_splits(m, b));
        if (s > need) need = s;
    }
    for (int t = 1; t <= m->MT; t++) {
        const size_t s = im_cuda_tq_scratch_bytes(1, t, m->nh_l, hd, tq_auto_splits(m->dev, 1, t, m->nkv_l, c.max_seq_len));
        if (s > need) need = s;
    }
    if (c.tq_bits == 16) {
        size_t n16 = 0;
        for (int b = 1; b <= c.max_batch; b++) n16 = std::max(n16, kv16_scratch_bytes(b, m->nh_l, kv16_auto_splits(m->dev, b, m->nkv_l, c.max_seq_len)));
        for (int t = 1; t <= m->MT; t++) n16 = std::max(n16, kv16_scratch_bytes(t, m->nh_l, kv16_auto_splits(m->dev, t, m->nkv_l, c.max_seq_len)));
        IM_TRY(m->alloc((void **)&m->kv16_scratch, n16));
        m->kv16_scratch_bytes = n16;
    }
    if (c.tq_bits != 16 && tq_prefill_scratch_bytes(m->nkv_l, c.max_seq_len) <= ((size_t)2 << 30))  // (longer caches: the per-token kernel)
        IM_TRY(m->alloc(&m->pf_dq, tq_prefill_scratch_bytes(m->nkv_l, c.max_seq_len)));
    IM_TRY(im_cuda_tq_reserve_scratch(m->tq, need));
    m->scratch_ref = reinterpret_cast<Tq *>(m->tq)->scratch;
    m->bytes += need + reinterpret_cast<Tq *>(m->tq)->const_bytes;
    IM_CUDA_CHECK(cudaDeviceSynchronize());
    IM_TRY(mega_prepare(m));
    m->finalized = true;
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_reset(im_model *m) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    for (char &u : m->slot_used) u = 0;
    return set_positions(m, 0);
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_truncate(im_model *m, int pos) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    if (pos < 0 || pos > m->slot_pos[0]) return fail(IM_ERR_BOUNDS, "truncate_to(%d) is outside the current sequence of %d tokens", pos, m->slot_pos[0]);
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    return set_positions(m, pos);
    IM_GUARD_END
}

// The final RMSNorm output the lm_head consumed in the last step (norm_out of
// crates/ironmill-inference/src/metal/pipeline.rs:176-226, decode_step_with_hidden / last_hidden_state), fp16 widened
// to f32: `rows` rows of hidden_size, one per sequence of that step in its order (row 0 for the single-sequence calls;
// after prefill_all_logits: one row per token of the last chunk).
IM_EXPORT int im_cuda_model_last_hidden_state(im_model *m, int rows, float *out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && out_host, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    const int cap = m->MT;
    if (rows < 1 || rows > cap) return fail(IM_ERR_BOUNDS, "rows must be in 1..%d, got %d", cap, rows);
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    const size_t n = (size_t)rows * m->cfg.hidden_size;
    std::vector<__half> tmp(n);
    IM_CUDA_CHECK(cudaMemcpyAsync(tmp.data(), m->norm_out, n * sizeof(__half), cudaMemcpyDeviceToHost, m->stream));
    IM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
    for (size_t i = 0; i < n; i++) out_host[i] = __half2float(tmp[i]);
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_seq_pos(const im_model *m) { return m && !m->slot_pos.empty() ? m->slot_pos[0] : 0; }
IM_EXPORT int im_cuda_model_max_seq_len(const im_model *m) { return m ? m->cfg.max_seq_len : 0; }
IM_EXPORT size_t im_cuda_model_memory_bytes(const im_model *m) { return m ? m->bytes : 0; }
// Timing of the whole-token decode kernel alone: `reps` launches back to back on the model's stream between two
// events (the sequence position is not advanced: every launch rewrites the same cache row), and the time CTA 0
// spent in each of the seven phases of a layer, averaged over the layers of the last launch, from the
// nanosecond-timer stamps it leaves at every grid barrier.  IM_ERR_STATE when the model does not use that kernel.
IM_EXPORT int im_cuda_model_token_kernel_profile(im_model *m, int reps, float *ms_per_launch, float *phase_us_7) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && reps >= 1 && ms_per_launch, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    if (!m->mega_ready) return fail(IM_ERR_STATE, "this model does not run the whole-token decode kernel");
    if (m->slot_pos[0] + 1 > m->cfg.max_seq_len) return fail(IM_ERR_BOUNDS, "no room for one more position");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    cudaStream_t st = m->stream;
    const im_model_config &c = m->cfg;
    IM_TRY(im_cuda_embedding_norm(m->tokens_dev, m->embed, m->layers[0].input_ln, m->norm_out, m->hidden, c.hidden_size, 1,
                                  (uint32_t)c.vocab_size, c.rms_eps, c.embed_scale != 0.0f ? c.embed_scale : 1.0f, st));
    IM_TRY(mega_launch(m->mega, m->dev, st));  // warm
    cudaEvent_t e0, e1;
    IM_CUDA_CHECK(cudaEventCreate(&e0));
    IM_CUDA_CHECK(cudaEventCreate(&e1));
    cudaEventRecord(e0, st);
    int rc = IM_OK;
    for (int i = 0; i < reps && rc == IM_OK; i++) rc = mega_launch(m->mega, m->dev, st);
    cudaEventRecord(e1, st);
    cudaMemcpyAsync(m->err_pin, m->dev->err_flag, sizeof(int), cudaMemcpyDeviceToHost, st);
    cudaError_t e = cudaStreamSynchronize(st);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    IM_TRY(rc);
    if (e != cudaSuccess) return fail(IM_ERR_CUDA, "whole-token kernel failed: %s", cudaGetErrorString(e));
    IM_TRY(step_error_check(m));
    *ms_per_launch = ms / (float)reps;
    if (phase_us_7) {
        const int L = c.num_layers, n = 7 * L + 2;
        std::vector<unsigned long long> t((size_t)n);
        IM_CUDA_CHECK(cudaMemcpy(t.data(), m->mega.trace, (size_t)n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        // t[0] start, t[k + 1] leaving barrier k (k = 0 .. 7L - 2), t[7L + 1] exit
        for (int j = 0; j < 7; j++) phase_us_7[j] = 0.0f;
        for (int l = 0; l < L; l++)
            for (int j = 0; j < 7; j++) {
                const int k = 7 * l + j;
                const unsigned long long end = k + 1 <= 7 * L - 1 ? t[(size_t)k + 1] : t[(size_t)7 * L + 1];
                const unsigned long long start = t[(size_t)k];
                phase_us_7[j] += (float)((double)(end - start) * 1e-3) / (float)L;
            }
    }
    return IM_OK;
    IM_GUARD_END
}

// Test hook of the error path: see the header.  The captured decode graphs hold the kernel's parameters by value, so
// they are dropped and the next step captures again.
IM_EXPORT int im_cuda_model_test_missing_ranks(im_model *m, int missing_ranks) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && (missing_ranks == 0 || missing_ranks == 1), "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    if (!m->mega_ready || !m->mega_capacity2 || m->world != 1)
        return fail(IM_ERR_STATE, "only for a single-GPU model loaded with decode_schedule = 2");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    IM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
    m->mega.world = 1 + missing_ranks;
    m->mega.xmail[1] = missing_ranks ? m->mega_phantom_mail : nullptr;  // where the stores "to the other rank" land
    for (auto &g : m->graphs) cudaGraphExecDestroy(g.second);
    m->graphs.clear();
    return IM_OK;
    IM_GUARD_END
}

// 1 when the row-split projections of a tensor-parallel model are summed by the one-shot peer-memory all-reduce,
// 0 when NCCL does it (single GPU: 0).
IM_EXPORT int im_cuda_model_tp_peer_allreduce(const im_model *m) { return m && m->xar.ok ? 1 : 0; }
IM_EXPORT int im_cuda_model_token_kernel(const im_model *m) { return m && m->mega_ready ? 1 : 0; }
IM_EXPORT int im_cuda_model_step_launches(const im_model *m) { return m ? m->launches_per_step : 0; }

IM_EXPORT size_t im_cuda_model_step_bytes(const im_model *m, int ctx, int batch) {
    if (!m || !m->finalized) return 0;
    const im_model_config &c = m->cfg;
    size_t b = 0;
    for (const Layer &L : m->layers) {
        for (const AffineWeight *w : {L.qkv, L.o, L.gate, L.up, L.down}) {
            b += (size_t)w->N * w->K * w->bits / 8 + (size_t)w->N * w->G * 4 + (w->awq ? (size_t)w->K * 2 : 0);
        }
        b += 2 * (size_t)c.hidden_size * 2;
        b += (size_t)batch * m->nkv_l * ctx * (2 * c.head_dim * c.tq_bits / 8 + (c.tq_bits == 16 ? 0 : 12));
    }
    b += (size_t)m->vocab_l * c.hidden_size * 2 + (size_t)c.hidden_size * 2;
    return b;
}

IM_EXPORT int im_cuda_model_prefill(im_model *m, const uint32_t *tokens_host, int n, float *logits_out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && tokens_host && logits_out_host, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_REQUIRE(n > 0, "prefill needs at least one token");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    return prefill_slot(m, 0, tokens_host, n, logits_out_host, nullptr);
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_prefill_all_logits(im_model *m, const uint32_t *tokens_host, int n, float *logits_out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && tokens_host && logits_out_host, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_REQUIRE(n > 0, "prefill needs at least one token");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    return prefill_slot(m, 0, tokens_host, n, nullptr, logits_out_host);
    IM_GUARD_END
}

// ---- continuous batching: BatchInferenceEngine (crates/ironmill-inference/src/engine.rs:121-131) -------------------
IM_EXPORT int im_cuda_model_seq_add(im_model *m, const uint32_t *tokens_host, int n, int *seq_id_out, float *logits_out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && tokens_host && seq_id_out, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_REQUIRE(n > 0, "a sequence needs at least one prompt token");
    int slot = -1;
    for (int s = 0; s < m->cfg.max_batch && slot < 0; s++)
        if (!m->slot_used[s]) slot = s;
    if (slot < 0) return fail(IM_ERR_BOUNDS, "all %d sequence slots are in use (max_batch)", m->cfg.max_batch);
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    set_one_pos_kernel<<<1, 1, 0, m->stream>>>(m->pos_dev, slot, 0);
    IM_CUDA_CHECK(cudaGetLastError());
    m->slot_pos[slot] = 0;
    int rc = prefill_slot(m, slot, tokens_host, n, logits_out_host, nullptr);
    if (rc != IM_OK) return rc;
    m->slot_used[slot] = 1;
    *seq_id_out = slot;
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_seq_remove(im_model *m, int seq_id) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    if (seq_id < 0 || seq_id >= m->cfg.max_batch || !m->slot_used[seq_id]) return fail(IM_ERR_INVALID, "no sequence %d", seq_id);
    m->slot_used[seq_id] = 0;   // the slot's cache rows are simply overwritten by the next tenant
    m->slot_pos[seq_id] = 0;
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_seq_position(const im_model *m, int seq_id) {
    if (!m || seq_id < 0 || seq_id >= (int)m->slot_pos.size() || !m->slot_used[seq_id]) return -1;
    return m->slot_pos[seq_id];
}

// One decode step for the listed sequences (any subset of the live ones, each at its own position): tokens_host[i] is
// appended to sequence seq_ids[i]; logits_out_host f32 [n, vocab] in the same order.
IM_EXPORT int im_cuda_model_batch_decode_step(im_model *m, const int *seq_ids, const uint32_t *tokens_host, int n, float *logits_out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && seq_ids && tokens_host && logits_out_host, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_REQUIRE(n >= 1 && n <= m->cfg.max_batch, "batch %d outside 1..max_batch (%d)", n, m->cfg.max_batch);
    for (int i = 0; i < n; i++) {
        const int s = seq_ids[i];
        if (s < 0 || s >= m->cfg.max_batch || !m->slot_used[s]) return fail(IM_ERR_INVALID, "no sequence %d", s);
        for (int j = 0; j < i; j++)
            if (seq_ids[j] == s) return fail(IM_ERR_INVALID, "sequence %d listed twice", s);
        if (m->slot_pos[s] + 1 > m->cfg.max_seq_len)
            return fail(IM_ERR_BOUNDS, "sequence %d: position %d + 1 exceeds max_seq_len %d", s, m->slot_pos[s], m->cfg.max_seq_len);
    }
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    cudaStream_t st = m->stream;
    memcpy(m->slot_pin, seq_ids, (size_t)n * sizeof(int));
    IM_CUDA_CHECK(cudaMemcpyAsync(m->slot_map, m->slot_pin, (size_t)n * sizeof(int), cudaMemcpyHostToDevice, st));
    cudaGraphExec_t g = nullptr;
    IM_TRY(get_graph(m, n, &g, true));
    memcpy(m->tokens_pin, tokens_host, (size_t)n * 4);
    IM_CUDA_CHECK(cudaMemcpyAsync(m->tokens_dev, m->tokens_pin, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    IM_CUDA_CHECK(cudaGraphLaunch(g, st));
    const __half *lg = m->world > 1 ? m->logits_all : m->logits;
    IM_CUDA_CHECK(cudaMemcpyAsync(m->logits_pin, lg, (size_t)n * m->cfg.vocab_size * 2, cudaMemcpyDeviceToHost, st));
    IM_CUDA_CHECK(cudaMemcpyAsync(m->err_pin, m->dev->err_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    IM_CUDA_CHECK(cudaStreamSynchronize(st));
    IM_TRY(step_error_check(m));
    for (int i = 0; i < n; i++) m->slot_pos[seq_ids[i]] += 1;
    logits_to_host(m, m->logits_pin, n, logits_out_host);
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_decode_step(im_model *m, const uint32_t *tokens_host, int batch, float *logits_out_host) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && tokens_host && logits_out_host, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_REQUIRE(batch >= 1 && batch <= m->cfg.max_batch, "batch %d outside 1..max_batch (%d)", batch, m->cfg.max_batch);
    int far = 0;
    for (int b = 0; b < batch; b++) far = m->slot_pos[b] > far ? m->slot_pos[b] : far;
    if (far + 1 > m->cfg.max_seq_len)
        return fail(IM_ERR_BOUNDS, "sequence position %d + 1 exceeds max_seq_len %d", far, m->cfg.max_seq_len);
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    cudaStream_t st = m->stream;
    cudaGraphExec_t g = nullptr;
    IM_TRY(get_graph(m, batch, &g));
    memcpy(m->tokens_pin, tokens_host, (size_t)batch * 4);
    IM_CUDA_CHECK(cudaMemcpyAsync(m->tokens_dev, m->tokens_pin, (size_t)batch * 4, cudaMemcpyHostToDevice, st));
    IM_CUDA_CHECK(cudaGraphLaunch(g, st));
    const __half *lg = m->world > 1 ? m->logits_all : m->logits;
    IM_CUDA_CHECK(cudaMemcpyAsync(m->logits_pin, lg, (size_t)batch * m->cfg.vocab_size * 2, cudaMemcpyDeviceToHost, st));
    IM_CUDA_CHECK(cudaMemcpyAsync(m->err_pin, m->dev->err_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    IM_CUDA_CHECK(cudaStreamSynchronize(st));
    IM_TRY(step_error_check(m));
    for (int b = 0; b < batch; b++) m->slot_pos[b] += 1;
    logits_to_host(m, m->logits_pin, batch, logits_out_host);
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_decode_greedy(im_model *m, const uint32_t *first_tokens_host, int batch, int n_steps,
                                          uint32_t *tokens_out_host, float *elapsed_ms_out) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && first_tokens_host, "bad argument");
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_REQUIRE(batch >= 1 && batch <= m->cfg.max_batch, "batch %d outside 1..max_batch (%d)", batch, m->cfg.max_batch);
    IM_REQUIRE(n_steps >= 0, "n_steps must be >= 0");
    int far = 0;
    for (int b = 0; b < batch; b++) far = m->slot_pos[b] > far ? m->slot_pos[b] : far;
    if (far + n_steps > m->cfg.max_seq_len)
        return fail(IM_ERR_BOUNDS, "sequence position %d + %d steps exceeds max_seq_len %d", far, n_steps, m->cfg.max_seq_len);
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    cudaStream_t st = m->stream;
    cudaGraphExec_t g = nullptr;
    IM_TRY(get_graph(m, batch, &g));
    memcpy(m->tokens_pin, first_tokens_host, (size_t)batch * 4);
    IM_CUDA_CHECK(cudaMemcpyAsync(m->tokens_dev, m->tokens_pin, (size_t)batch * 4, cudaMemcpyHostToDevice, st));
    IM_CUDA_CHECK(cudaMemsetAsync(m->step_dev, 0, 4, st));
    cudaEvent_t e0, e1;
    IM_CUDA_CHECK(cudaEventCreate(&e0));
    IM_CUDA_CHECK(cudaEventCreate(&e1));
    cudaEventRecord(e0, st);
    for (int i = 0; i < n_steps; i++) {
        cudaError_t e = cudaGraphLaunch(g, st);
        if (e != cudaSuccess) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            return fail(IM_ERR_CUDA, "graph launch failed: %s", cudaGetErrorString(e));
        }
    }
    cudaEventRecord(e1, st);
    cudaMemcpyAsync(m->err_pin, m->dev->err_flag, sizeof(int), cudaMemcpyDeviceToHost, st);
    cudaError_t e = cudaStreamSynchronize(st);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return fail(IM_ERR_CUDA, "decode loop failed: %s", cudaGetErrorString(e));
    IM_TRY(step_error_check(m));
    for (int b = 0; b < batch; b++) m->slot_pos[b] += n_steps;
    if (elapsed_ms_out) *elapsed_ms_out = ms;
    if (tokens_out_host && n_steps > 0)
        IM_CUDA_CHECK(cudaMemcpy2D(tokens_out_host, (size_t)batch * 4, m->tok_hist, (size_t)m->cfg.max_batch * 4, (size_t)batch * 4, n_steps,
                                   cudaMemcpyDeviceToHost));
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_model_profile_step(im_model *m, int batch, float *ms_by_category, int n_categories) {
    IM_GUARD_BEGIN
    IM_REQUIRE(m && ms_by_category && n_categories >= kCatCount, "bad argument (need %d categories)", (int)kCatCount);
    if (!m->finalized) return fail(IM_ERR_STATE, "model not loaded");
    IM_REQUIRE(batch >= 1 && batch <= m->cfg.max_batch, "batch %d outside 1..max_batch (%d)", batch, m->cfg.max_batch);
    for (int b = 0; b < batch; b++)
        if (m->slot_pos[b] + 1 > m->cfg.max_seq_len) return fail(IM_ERR_BOUNDS, "no room for one more position");
    IM_CUDA_CHECK(cudaSetDevice(m->dev->ordinal));
    cudaStream_t st = m->stream;
    const int splits = decode_splits(m, batch);
    IM_TRY(forward(m, batch, 1, splits, st, nullptr));  // warm
    Prof prof;
    prof.st = st;
    prof.mark(-1);
    int rc = forward(m, batch, 1, splits, st, nullptr, &prof);
    cudaError_t e = cudaStreamSynchronize(st);
    for (int i = 0; i < n_categories; i++) ms_by_category[i] = 0.0f;
    if (rc == IM_OK && e == cudaSuccess)
        for (size_t i = 1; i < prof.ev.size(); i++) {
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, prof.ev[i - 1], prof.ev[i]);
            ms_by_category[prof.cat[i]] += ms;
        }
    for (cudaEvent_t ev : prof.ev) cudaEventDestroy(ev);
    if (rc != IM_OK) return rc;
    if (e != cudaSuccess) return fail(IM_ERR_CUDA, "profile step failed: %s", cudaGetErrorString(e));
    return IM_OK;
    IM_GUARD_END
}

// Host-only helpers of the tensor-parallel loader, exported so that the shard arithmetic can be checked on a
// machine without a GPU.  `suffix` is the part of the tensor name after "model.layers.<i>.".
IM_EXPORT int im_cuda_tp_shard_rect(const im_model_config *cfg, const char *suffix, int *r0, int *nr, int *c0, int *nc) {
    IM_GUARD_BEGIN
    IM_REQUIRE(cfg && suffix && r0 && nr && c0 && nc, "bad argument");
    int en, ek;
    if (shard_rect(*cfg, suffix, r0, nr, c0, nc, &en, &ek) != IM_OK) return fail(IM_ERR_INVALID, "unknown projection '%s'", suffix);
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_tp_shard_affine(const void *qdata_host, const void *scales_host, const void *zeros_host, int param_dtype,
                                      const void *awq_f16_host, int N, int K, int group_size, int bit_width, int r0, int nr, int c0,
                                      int nc, void *q_out, void *scales_out, void *zeros_out, void *awq_out) {
    IM_GUARD_BEGIN
    IM_REQUIRE(qdata_host && scales_host && zeros_host && q_out && scales_out && zeros_out, "bad argument");
    HostAffine h;
    IM_TRY(slice_affine(&h, qdata_host, scales_host, zeros_host, param_dtype, awq_f16_host, N, K, group_size, bit_width, r0, nr, c0, nc));
    memcpy(q_out, h.q.data(), h.q.size());
    if (h.param_f32) {
        memcpy(scales_out, h.s.data(), h.s.size() * 4);
        memcpy(zeros_out, h.z.data(), h.z.size() * 4);
    } else {
        memcpy(scales_out, h.s16.data(), h.s16.size() * 2);
        memcpy(zeros_out, h.z16.data(), h.z16.size() * 2);
    }
    if (awq_out && !h.awq.empty()) memcpy(awq_out, h.awq.data(), h.awq.size() * 2);
    return IM_OK;
    IM_GUARD_END
}
