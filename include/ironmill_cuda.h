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

/* Dense fp16 matvec y = W x (lm_head): matvec
 * (.../shaders/linear/matvec.metal:30-84; crates/ironmill-inference/src/metal/pipeline.rs:1159-1174).
 * w_dev fp16 [N,K] row-major, x_dev fp16 [B,K], y_dev fp16 [B,N]. */
int im_cuda_matvec_f16(const void *w_dev, const void *x_dev, void *y_dev, int N, int K, int B, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* IRONMILL_CUDA_H */
