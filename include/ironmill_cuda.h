/*
 * ironmill_cuda.h - C ABI of the B200 (sm_100a) decode backend for ironmill.
 *
 * This is the boundary a Rust `ironmill-cuda-sys` crate binds, in the place
 * `ironmill-metal-sys` takes for the Metal backend.  Conventions follow the
 * reference's existing C API (docs/C_API.md:98-126): opaque handles, an `int`
 * status (0 = ok, negative = error), a thread-local message readable through
 * im_cuda_last_error(), `*_free(NULL)` is a no-op, nothing unwinds across the
 * boundary.
 *
 * Pointers named `*_dev` are CUDA device pointers of the current device;
 * pointers named `*_host` are ordinary host memory.  `stream` is a
 * `cudaStream_t` passed as `void*` (NULL = the legacy default stream).  All fp16
 * tensors are IEEE binary16, row-major.  Kernel entry points are asynchronous on
 * `stream` unless they take host pointers.
 *
 * Each declaration cites the reference interface it stands in for
 * (file:line relative to the reference project root).
 */
#ifndef IRONMILL_CUDA_H
#define IRONMILL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  Mirrors the split of MetalSysError
 * (crates/ironmill-metal-sys/src/error.rs:5-41) and InferenceError
 * (crates/ironmill-inference/src/engine.rs:17-58). */
#define IM_OK 0
#define IM_ERR_INVALID (-1)   /* InvalidArgument */
#define IM_ERR_CUDA (-2)      /* CommandBuffer / runtime error from CUDA */
#define IM_ERR_ALLOC (-3)     /* BufferAllocation / Allocation */
#define IM_ERR_BOUNDS (-4)    /* sequence or buffer range exceeded */
#define IM_ERR_TIMEOUT (-5)   /* a bounded device-side wait ran out */
#define IM_ERR_NCCL (-6)      /* collective failed */
#define IM_ERR_STATE (-7)     /* NotLoaded / wrong call order */
#define IM_ERR_NO_DEVICE (-8) /* NoDevice */

/* Thread-local message of the last failing call on this thread ("" if none). */
const char *im_cuda_last_error(void);

/* ABI version of this header (bumped on incompatible change). */
int im_cuda_abi_version(void);

/* ------------------------------------------------------------------ device
 * MetalDevice::system_default / create_buffer / current_allocated_size
 * (crates/ironmill-metal-sys/src/device.rs:74-260,395). */
typedef struct im_device im_device;
typedef struct im_buffer im_buffer;

int im_cuda_device_count(int *count_out);
int im_cuda_device_open(int ordinal, im_device **out);
void im_cuda_device_free(im_device *dev);
int im_cuda_device_ordinal(const im_device *dev);
int im_cuda_device_name(const im_device *dev, char *buf, size_t buf_len);
int im_cuda_device_sm_count(const im_device *dev);
/* Bytes currently allocated through this device handle (buffers, weights, models). */
size_t im_cuda_device_allocated_bytes(const im_device *dev);
int im_cuda_device_synchronize(im_device *dev);
/* Synchronises and reports IM_ERR_TIMEOUT if a kernel gave up a bounded device-side wait since the last
 * check (the counterpart of the command-buffer status check,
 * crates/ironmill-inference/src/metal/pipeline.rs:1209-1213). */
int im_cuda_device_check_error(im_device *dev);

/* MetalBuffer::{length, write_bytes, read_bytes} with bounds checks
 * (crates/ironmill-metal-sys/src/buffer.rs:42-158).  Buffers are device-private:
 * the host reaches them only through upload/download. */
int im_cuda_buffer_alloc(im_device *dev, size_t bytes, im_buffer **out);
int im_cuda_buffer_alloc_with_data(im_device *dev, const void *src_host, size_t bytes, im_buffer **out);
void im_cuda_buffer_free(im_buffer *buf);
size_t im_cuda_buffer_length(const im_buffer *buf);
void *im_cuda_buffer_ptr(const im_buffer *buf);
int im_cuda_buffer_upload(im_buffer *buf, size_t offset, const void *src_host, size_t bytes);
int im_cuda_buffer_download(const im_buffer *buf, size_t offset, void *dst_host, size_t bytes);

/* ------------------------------------------------------------------ quantize
 * Per-group affine quantization + INT4 packing on the GPU, bit-exact with
 * quantize_affine / emit_per_group / pack_int4
 * (crates/mil-rs/src/ir/passes/affine_quantize.rs:256-298,420-453,
 *  crates/mil-rs/src/ir/passes/int4_pack.rs:20-34) and with the AWQ pre-scale of
 * crates/ironmill-compile/src/weights/quantized.rs:912-947.
 * w_dev fp16 [rows,K]; awq_dev fp16 [K] or NULL; bit_width 4 or 8.
 * packed_dev: ceil(rows*K/2) bytes (4-bit, low nibble first over the flattened
 * stream) or rows*K bytes (8-bit).  scales_dev / zps_dev f32 [rows, ceil(K/group)]. */
int im_cuda_quantize_affine(const void *w_dev, const void *awq_dev, size_t rows, size_t K,
                            int group_size, int bit_width, void *packed_dev, float *scales_dev,
                            float *zps_dev, void *stream);

/* ------------------------------------------------------------------ weights
 * GPU-resident affine-quantized weight: AffineQuantizedWeight + load_weight_buffer
 * (crates/ironmill-inference/src/metal/weights.rs:129-147,1036-1114).
 * Scales/zero-points arrive as the bundle stores them (f32 or fp16, see
 * param_dtype) and are converted to fp16 round-to-nearest-even like
 * convert_params_to_f16 (crates/ironmill-core/src/dequant.rs:305-345); the
 * loader then repacks them into the interleaved (scale, zero) tiles the
 * kernels stream.  qdata: [N, K/2] (4-bit) or [N, K] (8-bit) row-major. */
typedef struct im_affine_weight im_affine_weight;
#define IM_DTYPE_F16 0
#define IM_DTYPE_F32 1

int im_cuda_affine_weight_create(im_device *dev, const void *qdata_host, const void *scales_host,
                                 const void *zeros_host, int param_dtype, const void *awq_f16_host,
                                 int N, int K, int group_size, int bit_width, im_affine_weight **out);
/* Same, with all inputs already on the device (params f32 or fp16 per param_dtype). */
int im_cuda_affine_weight_create_dev(im_device *dev, const void *qdata_dev, const void *scales_dev,
                                     const void *zeros_dev, int param_dtype, const void *awq_f16_dev,
                                     int N, int K, int group_size, int bit_width, void *stream,
                                     im_affine_weight **out);
void im_cuda_affine_weight_free(im_affine_weight *w);
size_t im_cuda_affine_weight_bytes(const im_affine_weight *w);
/* Standalone (q - z) * s dequant to fp16 [N,K]: int4_dequantize
 * (crates/ironmill-inference/src/metal/shaders/quantized/int4_dequant.metal:16-47),
 * dequant_affine (crates/ironmill-core/src/dequant.rs:85-180). */
int im_cuda_affine_weight_dequant(const im_affine_weight *w, void *out_f16_dev, void *stream);

/* ------------------------------------------------------------------ matvec family
 * y[b,n] = sum_k (x[b,k] / awq[k]) * (q[n,k] - z[n,g]) * s[n,g]  -> fp16.
 * superblock_matvec_int4 / _int8
 * (crates/ironmill-inference/src/metal/shaders/quantized/affine_matvec.metal:16-111,123-189;
 *  dispatch crates/ironmill-inference/src/metal/projection.rs:227-312).
 * x_dev fp16 [B,K], y_dev fp16 [B,N], 1 <= B <= 64. */
int im_cuda_matvec_affine(const im_affine_weight *w, const void *x_dev, void *y_dev, int B, void *stream);
/* Host-buffer form of the same call: copies x in, runs, copies y out, synchronises. */
int im_cuda_matvec_affine_host(const im_affine_weight *w, const void *x_host, void *y_host, int B);

/* out[b,n] = f16( silu(gate[n].x) * (up[n].x) ), dots kept in f32:
 * superblock_batched_affine_matvec_int4 + superblock_fused_ffn_gate_up_act_int4
 * (.../shaders/quantized/affine_batched.metal:5-91, affine_fused.metal:9-108;
 *  crates/ironmill-inference/src/metal/ffn.rs:25-87).  gate and up are [I,K] weights
 * that share x (and the AWQ vector of `gate`). */
int im_cuda_ffn_gate_up_act(const im_affine_weight *gate, const im_affine_weight *up, const void *x_dev,
                            void *out_dev, int B, void *stream);

/* r = a + b; y[n] = f16(rms_inv * sum_k (r_k gamma_k / awq_k) w[n,k]);
 * residual_out = f16(r); normed_out = f16(r * rms_inv * gamma)  (either may be NULL):
 * superblock_fused_residual_norm_affine_matvec_int4
 * (.../shaders/norm/superblock_fused_norm.metal:21-124; encode_end_of_layer_residual,
 *  crates/ironmill-inference/src/metal/attention.rs:616-702).  a,b fp16 [B,K]. */
int im_cuda_fused_residual_norm_matvec(const im_affine_weight *w, const void *a_dev, const void *b_dev,
                                       const void *gamma_dev, float eps, void *y_dev,
                                       void *residual_out_dev, void *normed_out_dev, int B, void *stream);

/* fused_residual_rms_norm followed by the fused gate+up+SiLU projection in one launch:
 * r = a + b; out[n] = f16( silu(rms_inv * gate[n].(r gamma / awq)) * (rms_inv * up[n].(r gamma / awq)) );
 * residual_out = f16(r), normed_out = f16(r * rms_inv * gamma) (either may be NULL for tiled INT4 weights).
 * Stands for the pair (.../shaders/norm/fused_residual_norm.metal:33-75, .../quantized/affine_fused.metal:9-108)
 * that the reference encodes back to back (crates/ironmill-inference/src/metal/pipeline.rs:887-905, ffn.rs:25-54);
 * the projection reads the unrounded normalised vector instead of its fp16 copy. */
int im_cuda_fused_residual_norm_ffn(const im_affine_weight *gate, const im_affine_weight *up, const void *a_dev,
                                    const void *b_dev, const void *gamma_dev, float eps, void *out_dev,
                                    void *residual_out_dev, void *normed_out_dev, int B, void *stream);

/* Dense fp16 matvec y = W x (lm_head): matvec
 * (.../shaders/linear/matvec.metal:30-84; crates/ironmill-inference/src/metal/pipeline.rs:1159-1174).
 * w_dev fp16 [N,K] row-major, x_dev fp16 [B,K], y_dev fp16 [B,N]. */
int im_cuda_matvec_f16(const void *w_dev, const void *x_dev, void *y_dev, int N, int K, int B, void *stream);
/* superblock_matmul_int4 (.../shaders/quantized/affine_matmul.metal:10-152), the dense-contraction case (prefill,
 * decode batches >= 16): y[M,N] = sum_k f16(x[m,k] / awq[k]) * f16((q - z) * s), f32 accumulation on the tcgen05
 * tensor cores, fp16 result.  INT4 group-128 weights; scratch_dev holds M*K halves (the scaled activations). */
int im_cuda_matmul_affine(const im_affine_weight *w, const void *x_dev, void *y_dev, int M, void *scratch_dev, void *stream);

/* ------------------------------------------------------------------ norms, embedding, RoPE
 * rms_norm (crates/ironmill-inference/src/metal/shaders/norm/normalization.metal:19-57):
 * out = f16(x * rsqrt(mean(x^2) + eps) * gamma), x fp16 [T,H]. */
int im_cuda_rms_norm(const void *x_dev, const void *gamma_dev, void *out_dev, int H, int T, float eps, void *stream);
/* fused_residual_rms_norm (.../shaders/norm/fused_residual_norm.metal:33-75):
 * residual = f16(a + b); normed from the unrounded f32 sum. */
int im_cuda_fused_residual_rms_norm(const void *a_dev, const void *b_dev, const void *gamma_dev, void *normed_dev,
                                    void *residual_dev, int H, int T, float eps, void *stream);
/* residual_add (.../shaders/elementwise/elementwise.metal:14-23). */
int im_cuda_residual_add(const void *a_dev, const void *b_dev, void *out_dev, size_t n, void *stream);
/* fused_embedding_norm (.../shaders/norm/fused_embedding_norm.metal:29-72): gather fp16 row * embed_scale
 * (zeros when token >= vocab) -> raw; RMSNorm * gamma -> normed.  tokens_dev u32 [T]. */
int im_cuda_embedding_norm(const uint32_t *tokens_dev, const void *table_dev, const void *gamma_dev, void *normed_dev,
                           void *raw_dev, int H, int T, uint32_t vocab, float eps, float embed_scale, void *stream);
/* fused_qk_norm_rope (.../shaders/norm/fused_qk_norm_rope.metal:43-124): per head RMSNorm with a [head_dim]
 * weight, then half-split RoPE over the first rotary_dim dims, in place.  q [T,nh,hd], k [T,nkv,hd];
 * cos/sin fp16 [max_pos, hd/2]; position of token t = seq_offset + t. */
int im_cuda_qk_norm_rope(void *q_dev, void *k_dev, const void *q_norm_w_dev, const void *k_norm_w_dev, const void *cos_dev,
                         const void *sin_dev, int nh, int nkv, int head_dim, int rotary_dim, int seq_offset, int T, float eps,
                         void *stream);
/* rope (.../shaders/rope/rope.metal:21-60): RoPE only (models without QK-norm), in place on qk [T,heads,hd]. */
int im_cuda_rope(void *qk_dev, const void *cos_dev, const void *sin_dev, int heads, int head_dim, int seq_offset, int T,
                 void *stream);
/* precompute_rope_cache (crates/ironmill-core/src/rope.rs:22-49): f64 on the host, rounded to fp16,
 * uploaded to cos_dev / sin_dev [max_pos, head_dim/2].  rotary_dim 0 = head_dim. */
int im_cuda_rope_table(int head_dim, int max_pos, double theta, int rotary_dim, void *cos_dev, void *sin_dev);

/* silu_gate (crates/ironmill-inference/src/metal/shaders/activation/activation.metal:15): out = f16(SiLU(gate) * up)
 * over n fp16 elements (n even), f32 inside; out may alias gate.  The prefill form of the FFN (metal/ffn.rs:58-150). */
int im_cuda_silu_mul(const void *gate_dev, const void *up_dev, void *out_dev, size_t n, void *stream);

/* ------------------------------------------------------------------ TurboQuant KV cache, 8 or 4 bits per element
 * Constants of MetalTurboQuantModel::new (crates/ironmill-inference/src/metal/turboquant/mod.rs:221-287):
 * rotation signs [hd] (+-1), QJL matrix [hd,hd] N(0,1), K codebook with 2^(bits-1) levels, V codebook with
 * 2^bits levels (lloyd_max_gaussian, crates/ironmill-inference/src/turboquant/codebook.rs:20-52). */
typedef struct im_tq im_tq;
/* Host computation of the Lloyd-Max codebook: levels[2^n_bits], bounds[2^n_bits - 1]. */
int im_cuda_tq_lloyd_max(int dim, int n_bits, float *levels_out_host, float *bounds_out_host);
/* Seeded sign vector and QJL matrix (stand-in for generate_rotation_signs / generate_qjl_matrix,
 * crates/ironmill-inference/src/turboquant/rotation.rs:13-49, whose values depend on the rand crate). */
int im_cuda_tq_generate(int head_dim, uint64_t seed, float *signs_out_host, float *qjl_out_host);
/* Codebook pointers may be NULL: they are then computed with im_cuda_tq_lloyd_max. */
int im_cuda_tq_create(im_device *dev, int head_dim, int n_bits, const float *signs_host, const float *qjl_host,
                      const float *k_levels_host, const float *k_bounds_host, const float *v_levels_host,
                      const float *v_bounds_host, im_tq **out);
void im_cuda_tq_free(im_tq *tq);
/* turboquant_cache_write (.../shaders/turboquant/turboquant.metal:52-170).  kv fp16 [nseq, T, nkv, hd];
 * cache u8 [nseq, nkv, max_seq, hd * n_bits / 8] (n_bits = 4: element 2i in the low nibble of byte i, 2i + 1 in the
 * high one, .../src/shaders/turboquant_helpers.metal:24-77); scale / r_norms f32 [nseq, nkv, max_seq]; write position
 * of token t of sequence s = (base_pos + pos_dev[s] + t) % max_seq (pos_dev may be NULL).  is_k selects the K form
 * ((n_bits - 1)-bit index | QJL sign in the top bit, residual norm) or the V form (n_bits-bit index). */
int im_cuda_tq_encode(const im_tq *tq, const void *kv_dev, int is_k, void *cache_dev, float *scale_dev, float *r_norms_dev,
                      int nseq, int nkv, int max_seq, int base_pos, const int *pos_dev, int T, void *stream);
/* turboquant_attention in split mode + fused_sdpa_reduce (.../turboquant/turboquant.metal:202-462,
 * .../attention/flash_decode.metal:163-215; dispatch crates/ironmill-inference/src/metal/attention.rs:394-489).
 * q, out fp16 [nseq, T, nh, hd]; causal length of token t = base_pos + pos_dev[s] + t + 1.
 * num_splits 0 = chosen from the device size and the sequence length.  The split partials live in
 * scratch memory owned by the handle (grown on demand; reserve it up front to keep this call
 * allocation-free). */
int im_cuda_tq_attention(im_tq *tq, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                         const float *k_scale_dev, const float *v_scale_dev, const float *k_rnorm_dev, float attn_scale,
                         void *out_dev, int nseq, int nh, int nkv, int max_seq, int base_pos, const int *pos_dev, int T,
                         int num_splits, void *stream);
/* One call for the whole attention block of a decode step, two launches + reduce instead of five:
 * (fused_qk_norm_rope | rope) on the q and k parts of a fused QKV row, turboquant_cache_write of K and V, the query
 * rotation that turboquant_attention starts with (done once per head here), then the split attention.
 * qkv_dev fp16 [nseq*T, qkv_stride] with q at 0, k at k_offset, v at v_offset (elements); norm weights NULL = plain
 * RoPE (Llama); qrot_dev f32 scratch [nseq*T, nh, 2, head_dim].  Same references as the separate entry points. */
int im_cuda_tq_fused_attention(im_tq *tq, const void *qkv_dev, int qkv_stride, int k_offset, int v_offset,
                               const void *q_norm_w_dev, const void *k_norm_w_dev, const void *cos_dev, const void *sin_dev,
                               int rotary_dim, float eps, void *k_cache_dev, void *v_cache_dev, float *k_scale_dev,
                               float *v_scale_dev, float *k_rnorm_dev, float attn_scale, float *qrot_dev, void *out_dev,
                               int nseq, int nh, int nkv, int max_seq, int base_pos, const int *pos_dev, int T,
                               int num_splits, void *stream);
/* im_cuda_tq_attention for callers that must not allocate.  (No counterpart in the reference: its Metal backend
 * sizes every buffer up front; this entry point exists for CUDA hosts that cannot call cudaMalloc when they need
 * attention - an arena-owning server, a plugin whose host forbids allocation after start-up, code that runs between
 * another component's graph capture and replay.)  It allocates nothing and calls nothing that allocates: the split
 * partials go into a 4 MiB array inside the library image, which every GPU that loads the library keeps until the
 * process exits.  Same arguments, kernels and results as im_cuda_tq_attention.  Limits and rules:
 *  - the split partials and the rotated queries, nseq * T * nh * (splits * 520 + 1024) bytes, must fit 4 MiB: with
 *    num_splits = 0 the library lowers its own split count until they do, a count given by the caller is refused with
 *    IM_ERR_BOUNDS and the numbers in the message;
 *  - the device of `tq` must be the current device;
 *  - the first call on a device looks the array's device address up (cudaGetSymbolAddress); make that first call
 *    before any stream capture;
 *  - all calls share the one array, which keeps whatever the last call left in it (nothing needs clearing: every
 *    split writes its whole partial before it is read); two calls whose kernels overlap on the GPU race. */
int im_cuda_tq_attention_static(const im_tq *tq, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                                const float *k_scale_dev, const float *v_scale_dev, const float *k_rnorm_dev, float attn_scale,
                                void *out_dev, int nseq, int nh, int nkv, int max_seq, int base_pos, const int *pos_dev, int T,
                                int num_splits, void *stream);
/* Prefill form for one sequence (T tokens at positions base_pos .. base_pos + T - 1, rows already in the cache, the
 * reference's turboquant_attention with token_count > 1, turboquant.metal:202-462): the cached rows are dequantised once
 * into dq_dev (im_cuda_tq_prefill_scratch_bytes(nkv, max_seq) bytes) and scored by a causal tensor-core pass.  Caches of
 * one sequence: [nkv, max_seq, ...].  Same results as im_cuda_tq_attention within its tolerance. */
size_t im_cuda_tq_prefill_scratch_bytes(int nkv, int max_seq);
int im_cuda_tq_prefill_attention(im_tq *tq, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev, const float *k_scale_dev,
                                 const float *v_scale_dev, const float *k_rnorm_dev, float attn_scale, void *out_dev, int nh, int nkv,
                                 int max_seq, int base_pos, int T, void *dq_dev, void *stream);
/* Scratch im_cuda_tq_attention needs for a launch: split partials (nseq*T*nh*splits*(head_dim+2) floats) plus the
 * rotated queries of its pre-pass (nseq*T*nh*2*head_dim floats).  The handle grows its scratch on demand. */
size_t im_cuda_tq_scratch_bytes(int nseq, int T, int nh, int head_dim, int splits);
int im_cuda_tq_reserve_scratch(im_tq *tq, size_t bytes);

/* ---- fp16 (unquantized) KV cache: the reference's path with TurboQuant off ----------------------------------------
 * (ironmill-inference/src/metal/attention.rs:491-612).  head_dim must be 128.
 * im_cuda_kv_scatter_f16 replaces kv_scatter (shaders/kv/kv_scatter.metal:20-42): proj fp16 [nseq*T, nkv, head_dim] is
 * written to cache fp16 [slots, nkv, max_seq, head_dim] at position (base_pos + pos_dev[slot] + t) % max_seq of the
 * token's sequence (slot_map_dev: optional sequence -> cache slot).
 * im_cuda_sdpa_f16 replaces fused_sdpa (shaders/attention/fused_sdpa.metal:52-251), prefill_attention_v2
 * (shaders/attention/attention.metal:571-750) and the pair fused_sdpa_split / fused_sdpa_reduce
 * (shaders/attention/flash_decode.metal:25-215): out[t, h] = softmax(scale * q[t, h] . K^T) V over the positions
 * 0 .. base_pos + pos_dev[seq] + t of the head's KV head (causal), fp16 in and out, f32 scores and sums.
 * q, out fp16 [nseq*T, nh, head_dim].  num_splits = 0 lets the library choose (1 = single pass); more than one split
 * needs scratch_dev of im_cuda_sdpa_f16_scratch_bytes(nseq, T, nh, splits) bytes. */
int im_cuda_kv_scatter_f16(const void *proj_dev, void *cache_dev, int nseq, int T, int nkv, int head_dim, int max_seq, int base_pos,
                           const int *pos_dev, const int *slot_map_dev, void *stream);
size_t im_cuda_sdpa_f16_scratch_bytes(int nseq, int T, int nh, int splits);
int im_cuda_sdpa_f16(im_device *dev, const void *q_dev, const void *k_cache_dev, const void *v_cache_dev, void *out_dev, int nseq, int nh,
                     int nkv, int head_dim, int max_seq, int base_pos, const int *pos_dev, int T, float scale, int num_splits,
                     void *scratch_dev, size_t scratch_bytes, void *stream);

/* ------------------------------------------------------------------ model-level engine
 * The CUDA counterpart of MetalInference behind the InferenceEngine trait
 * (crates/ironmill-inference/src/engine.rs:72-114; crates/ironmill-inference/src/metal/engine.rs:122-270,
 *  loading.rs:483-518, pipeline.rs:228-1313).  One call = one whole token (or prompt chunk): the decode
 * step is captured once per batch size into a CUDA graph and replayed.
 *
 * Config mirrors ModelConfig (crates/mil-rs/src/weights.rs:57-97) + MetalConfig
 * (crates/ironmill-inference/src/metal/config.rs:270-299).  Zero in an optional field selects the default
 * named beside it. */
typedef struct im_model im_model;
typedef struct im_model_config {
    int num_layers, hidden_size, intermediate_size, num_heads, num_kv_heads, head_dim, vocab_size;
    int max_seq_len;          /* MetalConfig.max_seq_len (default 2048) */
    int max_batch;            /* sequences decoded in lockstep (default 1) */
    float rms_eps;
    float attn_scale;         /* 0 = 1/sqrt(head_dim) (crates/mil-rs/src/weights.rs:210-217) */
    float embed_scale;        /* 0 = 1.0 */
    double rope_theta;
    int rotary_dim;           /* 0 = head_dim */
    int qk_norm;              /* 1: q_norm / k_norm weights present (Qwen3) */
    int tie_word_embeddings;  /* 1: lm_head = embedding table */
    int tq_bits;              /* MetalConfig.n_bits: TurboQuant KV bits, 8 or 4 (0 = 8); 16 = MetalConfig.enable_turboquant
                               * off: an unquantized fp16 KV cache (kv_scatter + fused_sdpa / FlashDecoding) */
    uint64_t rotation_seed;   /* MetalConfig.rotation_seed (default 42) */
    int tp_world, tp_rank;    /* tensor parallel group (0/0 = single GPU) */
    int prefill_chunk_size;   /* MetalConfig.prefill_chunk_size: tokens per prefill forward (0 = 2048, the most; never more
                               * than max_seq_len; the activation buffers are sized for it) */
    int decode_schedule;      /* batch-1 decode: 0 = the whole-token kernel whenever the model fits it, 1 = always the
                                 graph of per-projection kernels, 2 = the whole-token kernel handing the o / down outputs on
                                 as tagged pairs instead of grid barriers (what tensor-parallel ranks do; one GPU: a way to
                                 run that code path) */
    int tp_collective;        /* tensor parallel: 0 = the library's peer-memory exchange when every rank could map its
                                 peers, 1 = NCCL all-reduce only */
    int wait_limit_ms;        /* patience of the device-side bounded waits (0 = 400 ms, 5 s under tensor parallelism) */
} im_model_config;

int im_cuda_model_create(im_device *dev, const im_model_config *cfg, im_model **out);
void im_cuda_model_free(im_model *m);
/* Tensors arrive under their Hugging Face names (crates/ironmill-inference/src/weight_loading.rs:163-426):
 * model.embed_tokens.weight, model.layers.{i}.input_layernorm.weight, .self_attn.{q,k,v,o}_proj.weight,
 * .self_attn.{q,k}_norm.weight, .post_attention_layernorm.weight, .mlp.{gate,up,down}_proj.weight,
 * model.norm.weight, lm_head.weight.  Each rank is handed the FULL tensor and keeps its shard. */
int im_cuda_model_load_dense(im_model *m, const char *name, const void *data_f16_host, size_t num_elements);
int im_cuda_model_load_affine(im_model *m, const char *name, const void *qdata_host, const void *scales_host,
                              const void *zeros_host, int param_dtype, const void *awq_f16_host, int N, int K,
                              int group_size, int bit_width);
/* Optional: rotation signs [hd] and QJL matrix [hd,hd]; otherwise generated from rotation_seed. */
int im_cuda_model_set_tq_constants(im_model *m, const float *signs_host, const float *qjl_host);
/* Tensor parallel: rank 0 makes an id (128 bytes), every rank passes the same bytes. */
int im_cuda_tp_unique_id(void *id_out_128_bytes);
int im_cuda_model_tp_init(im_model *m, const void *id_128_bytes);
/* Host-only pieces of the tensor-parallel loader (no GPU needed): the rectangle [r0,r0+nr) x [c0,c0+nc) of a full
 * projection that rank cfg->tp_rank keeps (`suffix` = tensor name after "model.layers.<i>."), and the cut itself
 * into caller buffers sized for the shard.  (Tensor parallelism has no counterpart in the reference.) */
int im_cuda_tp_shard_rect(const im_model_config *cfg, const char *suffix, int *r0, int *nr, int *c0, int *nc);
int im_cuda_tp_shard_affine(const void *qdata_host, const void *scales_host, const void *zeros_host, int param_dtype,
                            const void *awq_f16_host, int N, int K, int group_size, int bit_width, int r0, int nr, int c0,
                            int nc, void *q_out, void *scales_out, void *zeros_out, void *awq_out);
/* Checks that every tensor arrived, repacks, allocates KV caches / RoPE tables / TurboQuant constants
 * (init_model_state, crates/ironmill-inference/src/metal/loading.rs:32-65). */
int im_cuda_model_finalize(im_model *m);
/* InferenceEngine::prefill / decode_step: logits_out_host f32 [vocab] (prefill: last token) or
 * [batch, vocab] (decode).  Tokens are host u32.  Sequence overflow returns IM_ERR_BOUNDS
 * (crates/ironmill-inference/src/metal/pipeline.rs:270-279). */
int im_cuda_model_prefill(im_model *m, const uint32_t *tokens_host, int n_tokens, float *logits_out_host);
int im_cuda_model_decode_step(im_model *m, const uint32_t *tokens_host, int batch, float *logits_out_host);
/* Greedy decoding kept on the device: n_steps graph replays, each feeding the arg-max token (last
 * maximal index, crates/ironmill-inference/src/sampling.rs:331-339) of the previous one.  first_tokens_host
 * [batch]; tokens_out_host u32 [n_steps, batch] (may be NULL); elapsed_ms_out = CUDA-event time of the loop. */
int im_cuda_model_decode_greedy(im_model *m, const uint32_t *first_tokens_host, int batch, int n_steps,
                                uint32_t *tokens_out_host, float *elapsed_ms_out);
/* BatchInferenceEngine (crates/ironmill-inference/src/engine.rs:121-131; the reference declares the trait and has no
 * implementor): sequences that come and go, each in one of max_batch cache slots with its own position.
 * seq_add prefills the prompt into a free slot and returns its id (logits_out_host, optional: f32 [vocab] of the last
 * prompt token); seq_remove frees the slot; batch_decode_step appends tokens_host[i] to sequence seq_ids[i] for any
 * subset of the live sequences, whatever their lengths, and returns f32 [n, vocab] in the same order.  The
 * single-sequence calls above work on slot 0 and the lockstep form of decode_step on slots 0 .. batch - 1:
 * use one interface or the other on a model.  im_cuda_model_reset frees every slot. */
int im_cuda_model_seq_add(im_model *m, const uint32_t *tokens_host, int n_tokens, int *seq_id_out, float *logits_out_host);
int im_cuda_model_seq_remove(im_model *m, int seq_id);
int im_cuda_model_seq_position(const im_model *m, int seq_id);   /* tokens in the sequence's cache; -1: no such sequence */
int im_cuda_model_batch_decode_step(im_model *m, const int *seq_ids, const uint32_t *tokens_host, int n, float *logits_out_host);
int im_cuda_model_reset(im_model *m);
int im_cuda_model_truncate(im_model *m, int pos);
/* Hidden state of the last step: the final RMSNorm output the lm_head consumed, fp16 widened to f32, `rows` rows of
 * hidden_size (row i = sequence i of that step; row 0 for the single-sequence calls).  Replaces
 * MetalInference::decode_step_with_hidden / last_hidden_state (ironmill-inference/src/metal/pipeline.rs:176-226), which
 * read the same buffer (norm_out) for the draft head of speculative decoding: call it right after decode_step. */
int im_cuda_model_last_hidden_state(im_model *m, int rows, float *out_host);
int im_cuda_model_seq_pos(const im_model *m);
int im_cuda_model_max_seq_len(const im_model *m);
size_t im_cuda_model_memory_bytes(const im_model *m);
/* Algorithmic bytes one decode step of this rank reads from HBM at context length ctx and the given batch:
 * packed codes + scales/zeros + AWQ vectors + fp16 lm_head rows + norm weights + batch * KV bytes. */
size_t im_cuda_model_step_bytes(const im_model *m, int ctx, int batch);
/* 1 when the row-split projections of a tensor-parallel model are summed by the library's one-shot all-reduce over
 * peer memory (CUDA IPC + NVLink stores, set up by im_cuda_model_tp_init; im_model_config.tp_collective = 1 keeps NCCL), 0 when NCCL's
 * all-reduce does it.  No counterpart in the reference (it has no tensor parallelism). */
int im_cuda_model_tp_peer_allreduce(const im_model *m);
/* 1 when batch-1 decode steps of this model run in the whole-token kernel (all layers in one cooperative launch), 0
 * when they run as a graph of per-projection kernels.  Under tensor parallelism the kernel of every rank exchanges the
 * partial sums of the row-split projections through peer memory and its barriers after those projections span all
 * ranks (im_model_config.decode_schedule = 1 keeps the per-kernel schedule). */
int im_cuda_model_token_kernel(const im_model *m);
/* Number of kernel launches in one captured decode step. */
int im_cuda_model_step_launches(const im_model *m);
/* Timing of the whole-token decode kernel (all layers of a batch-1 step in one launch) by itself: the counterpart of
 * MetalConfig.kernel_timing for that kernel (crates/ironmill-inference/src/metal/pipeline.rs:353-422).
 * ms_per_launch: average of `reps` back-to-back launches between two events on the model's stream;
 * phase_us_7 (optional, 7 floats): microseconds per layer in QKV, RoPE + cache write, attention, split reduction,
 * o, gate/up, down.  IM_ERR_STATE when the model does not use that kernel (batch > 1 only, tensor parallel,
 * non-INT4 weights, decode_schedule = 1). */
int im_cuda_model_token_kernel_profile(im_model *m, int reps, float *ms_per_launch, float *phase_us_7);
/* InferenceEngine::prefill_all_logits (crates/ironmill-inference/src/metal/pipeline.rs:38-70, the perplexity path):
 * like im_cuda_model_prefill, but logits_out_host receives f32 [n_tokens, vocab], one row per prompt token. */
int im_cuda_model_prefill_all_logits(im_model *m, const uint32_t *tokens_host, int n_tokens, float *logits_out_host);
/* Host-side fault injection for tests of the error path (no counterpart in the reference).  Only for a model loaded
 * with decode_schedule = 2 on one GPU: with missing_ranks = 1 the whole-token kernel also waits for the partial sums
 * of a rank that does not exist, so its bounded wait runs out after wait_limit_ms, the kernel finishes, and the step
 * returns IM_ERR_TIMEOUT; 0 restores normal operation.  Nothing faults or hangs: a wait gives up and sets a word. */
int im_cuda_model_test_missing_ranks(im_model *m, int missing_ranks);
/* Per-category GPU time of one eager decode step at the current position, which is not advanced
 * (MetalConfig.kernel_timing, crates/ironmill-inference/src/metal/pipeline.rs:353-422,1215-1234).
 * ms_by_category[11]: embed, qkv projection, rope, kv write, attention, o projection, residual+norm,
 * gate+up+act, down projection, collectives, final norm + lm_head. */
int im_cuda_model_profile_step(im_model *m, int batch, float *ms_by_category, int n_categories);

#ifdef __cplusplus
}
#endif
#endif /* IRONMILL_CUDA_H */
