/*
 * CPU oracle for the quantized-decode hot path of jafreck/ironmill.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's CPU Rust code (quantize / pack / dequant / codebook / RoPE table)
 * and of the arithmetic of its Metal shaders (matvec family, norms, RoPE,
 * TurboQuant encode and decode attention).  It is the checker the CUDA path
 * is compared against and the timed "port" CPU baseline; nothing in the
 * product library links, imports or calls it.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference project root).  Compile with -ffp-contract=off so that no
 * multiply-add is fused: the bit-exact gates (quantize, TurboQuant encode)
 * depend on the operation order written here.
 *
 * Parity pins: the known-answer vectors of the reference's own unit tests for
 * quantize_affine, pack_int4, dequant_affine, the codebook properties and the
 * RoPE table are replayed against these functions by tests/test_oracle_*.py.
 * The values of the TurboQuant rotation signs and QJL matrix come from the
 * `rand` 0.10 crate (StdRng = ChaCha12) in the reference and are not pinned by
 * any reference test; here they are inputs (parity unpinned for their values,
 * pinned for everything computed from them).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t h) { f16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f2h(float f) { f16 v = (f16)f; uint16_t h; memcpy(&h, &v, 2); return h; }
static inline uint16_t d2h(double f) { f16 v = (f16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

#define EXPORT __attribute__((visibility("default")))

EXPORT int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------
 * Affine quantize (bit-exact gate)
 * crates/mil-rs/src/ir/passes/affine_quantize.rs:256-298 (quantize_affine)
 * ---------------------------------------------------------------------- */
EXPORT void orc_quantize_affine(const float *v, size_t n, float qmax,
                                uint8_t *q, float *scale_out, float *zp_out) {
    if (n == 0) { *scale_out = 1.0f; *zp_out = 0.0f; return; }
    float mn = INFINITY, mx = -INFINITY;
    for (size_t i = 0; i < n; i++) {
        float x = v[i];
        if (isfinite(x)) {
            if (x < mn) mn = x;
            if (x > mx) mx = x;
        }
    }
    if (!isfinite(mn) || !isfinite(mx)) {
        memset(q, 0, n);
        *scale_out = 1.0f; *zp_out = 0.0f;
        return;
    }
    float scale, zp;
    if (fabsf(mx - mn) < FLT_EPSILON) {
        scale = 1.0f;
        zp = roundf(-mn);
    } else {
        scale = (mx - mn) / qmax;
        zp = roundf(-mn / scale);
    }
    for (size_t i = 0; i < n; i++) {
        float t = roundf(v[i] / scale + zp);
        /* Rust f32::clamp keeps NaN; `as u8` then saturates NaN to 0. */
        if (t != t) { q[i] = 0; continue; }
        if (t < 0.0f) t = 0.0f;
        if (t > qmax) t = qmax;
        q[i] = (uint8_t)t;
    }
    *scale_out = scale; *zp_out = zp;
}

/* crates/mil-rs/src/ir/passes/affine_quantize.rs:300-312 (dequantize_affine,
 * the f32 helper the reference's round-trip tests use). */
EXPORT void orc_dequantize_affine_f32(const uint8_t *q, size_t n, float scale, float zp, float *out) {
    for (size_t i = 0; i < n; i++) out[i] = ((float)q[i] - zp) * scale;
}

/* Per-group walk over a row-major [rows, K] tensor, groups along the last axis,
 * last group may be partial.
 * crates/mil-rs/src/ir/passes/affine_quantize.rs:420-453 (emit_per_group),
 * crates/ironmill-compile/src/weights/quantized.rs:408-466,852-900.
 * Input is fp16 widened exactly to f32 (crates/mil-rs/.../tensor_utils.rs:34-42);
 * with awq != NULL the f32 weight is first multiplied by f32(awq[col])
 * (quantized.rs:925-940).  codes: one byte per element. */
EXPORT void orc_quantize_groups_f16(const uint16_t *w, size_t rows, size_t K, size_t gs,
                                    int bits, const uint16_t *awq,
                                    uint8_t *codes, float *scales, float *zps, int threads) {
    const float qmax = bits == 4 ? 15.0f : 255.0f;
    const size_t ng = (K + gs - 1) / gs;
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for (size_t r = 0; r < rows; r++) {
        float *buf = (float *)malloc(sizeof(float) * gs);
        for (size_t g = 0; g < ng; g++) {
            size_t c0 = g * gs, c1 = c0 + gs < K ? c0 + gs : K;
            for (size_t c = c0; c < c1; c++) {
                float x = h2f(w[r * K + c]);
                if (awq) x = x * h2f(awq[c]);
                buf[c - c0] = x;
            }
            orc_quantize_affine(buf, c1 - c0, qmax, codes + r * K + c0,
                                &scales[r * ng + g], &zps[r * ng + g]);
        }
        free(buf);
    }
}

/* Same walk over f32 input (the pass operates on f32 slices). */
EXPORT void orc_quantize_groups_f32(const float *w, size_t rows, size_t K, size_t gs, int bits,
                                    uint8_t *codes, float *scales, float *zps) {
    const float qmax = bits == 4 ? 15.0f : 255.0f;
    const size_t ng = (K + gs - 1) / gs;
    for (size_t r = 0; r < rows; r++)
        for (size_t g = 0; g < ng; g++) {
            size_t c0 = g * gs, c1 = c0 + gs < K ? c0 + gs : K;
            orc_quantize_affine(w + r * K + c0, c1 - c0, qmax, codes + r * K + c0,
                                &scales[r * ng + g], &zps[r * ng + g]);
        }
}

/* crates/mil-rs/src/ir/passes/int4_pack.rs:20-34 (pack_int4): low nibble first,
 * odd tail padded with 0, values masked to 4 bits. */
EXPORT void orc_pack_int4(const uint8_t *v, size_t n, uint8_t *out) {
    for (size_t i = 0, o = 0; i < n; i += 2, o++) {
        uint8_t lo = v[i] & 0x0F;
        uint8_t hi = (i + 1 < n) ? (v[i + 1] & 0x0F) : 0;
        out[o] = (uint8_t)((hi << 4) | lo);
    }
}

/* crates/mil-rs/src/ir/passes/int4_pack.rs:40-55 (unpack_int4). */
EXPORT void orc_unpack_int4(const uint8_t *packed, size_t count, uint8_t *out) {
    for (size_t i = 0; i < count; i++) {
        uint8_t b = packed[i / 2];
        out[i] = (i % 2 == 0) ? (b & 0x0F) : ((b >> 4) & 0x0F);
    }
}

/* crates/ironmill-core/src/dequant.rs:305-345 (convert_params_to_f16): RNE. */
EXPORT void orc_f32_to_f16(const float *src, size_t n, uint16_t *dst) {
    for (size_t i = 0; i < n; i++) dst[i] = f2h(src[i]);
}
EXPORT void orc_f16_to_f32(const uint16_t *src, size_t n, float *dst) {
    for (size_t i = 0; i < n; i++) dst[i] = h2f(src[i]);
}

static inline float read_q(const uint8_t *qd, size_t i, int bits) {
    if (bits == 4) {
        uint8_t b = qd[i / 2];
        return (float)((i % 2 == 0) ? (b & 0x0F) : ((b >> 4) & 0x0F));
    }
    return (float)qd[i];
}

/* crates/ironmill-core/src/dequant.rs:85-180 (dequant_affine).
 * mode 0: per-group along the last axis (gs), scale/zp [rows, ceil(K/gs)]
 * mode 1: per-axis (axis index `axis`, dims given by outer/axis_size/stride)
 * mode 2: per-tensor.  scale/zp element type: f32 when *_is_f32 else fp16.
 * Output fp16 = f16((q - z) * s). */
EXPORT void orc_dequant_affine(const uint8_t *qd, const void *scale, const void *zp,
                               int scale_is_f32, int zp_is_f32, int mode,
                               size_t total, size_t K, size_t gs,
                               size_t axis_size, size_t stride, int bits, uint16_t *out) {
#define RD(p, isf32, i) ((isf32) ? ((const float *)(p))[i] : h2f(((const uint16_t *)(p))[i]))
    if (mode == 0) {
        size_t rows = total / K, ng = (K + gs - 1) / gs;
        for (size_t r = 0; r < rows; r++)
            for (size_t c = 0; c < K; c++) {
                size_t pi = r * ng + c / gs;
                float s = RD(scale, scale_is_f32, pi), z = RD(zp, zp_is_f32, pi);
                out[r * K + c] = f2h((read_q(qd, r * K + c, bits) - z) * s);
            }
    } else if (mode == 1) {
        for (size_t i = 0; i < total; i++) {
            size_t ai = (i / stride) % axis_size;
            float s = RD(scale, scale_is_f32, ai), z = RD(zp, zp_is_f32, ai);
            out[i] = f2h((read_q(qd, i, bits) - z) * s);
        }
    } else {
        float s = RD(scale, scale_is_f32, 0), z = RD(zp, zp_is_f32, 0);
        for (size_t i = 0; i < total; i++) out[i] = f2h((read_q(qd, i, bits) - z) * s);
    }
#undef RD
}

/* ------------------------------------------------------------------------
 * Matvec family (tolerance gate)
 * ---------------------------------------------------------------------- */

/* Decode projection, spec form y[n] = sum_k (x[k]/awq[k]) * (q[n,k]-z[n,g]) * s[n,g].
 * crates/ironmill-inference/src/metal/shaders/quantized/affine_matvec.metal:16-111,123-189
 * with the (q - z) * s dequant of crates/ironmill-core/src/dequant.rs:129-139
 * (the int4 shader's additive-bias reading of the zeros buffer is not reproduced).
 * x [B,K] fp16, y [B,N] fp16; f32 accumulation in ascending k. */
EXPORT void orc_matvec_affine(const uint8_t *qd, const uint16_t *scales, const uint16_t *zeros,
                              const uint16_t *awq, const uint16_t *x, uint16_t *y,
                              size_t N, size_t K, size_t gs, int bits, size_t B, int threads) {
    const size_t ng = (K + gs - 1) / gs;
    (void)threads;
    float *xs = (float *)malloc(sizeof(float) * B * K);
    for (size_t b = 0; b < B; b++)
        for (size_t k = 0; k < K; k++) {
            float v = h2f(x[b * K + k]);
            if (awq) v = v / h2f(awq[k]);
            xs[b * K + k] = v;
        }
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for (size_t n = 0; n < N; n++) {
        for (size_t b = 0; b < B; b++) {
            float acc = 0.0f;
            for (size_t k = 0; k < K; k++) {
                size_t pi = n * ng + k / gs;
                float w = (read_q(qd, n * K + k, bits) - h2f(zeros[pi])) * h2f(scales[pi]);
                acc += xs[b * K + k] * w;
            }
            y[b * N + n] = f2h(acc);
        }
    }
    free(xs);
}

/* Prefill / batched form: A' = f16(A/awq), Wd = f16((q-z)s), C = f16(sum f32(A')f32(Wd)).
 * crates/ironmill-inference/src/metal/shaders/quantized/affine_matmul.metal:10-152,155-290 */
EXPORT void orc_matmul_affine(const uint8_t *qd, const uint16_t *scales, const uint16_t *zeros,
                              const uint16_t *awq, const uint16_t *a, uint16_t *c,
                              size_t M, size_t N, size_t K, size_t gs, int bits, int threads) {
    const size_t ng = (K + gs - 1) / gs;
    (void)threads;
    float *as = (float *)malloc(sizeof(float) * M * K);
    for (size_t m = 0; m < M; m++)
        for (size_t k = 0; k < K; k++) {
            float v = h2f(a[m * K + k]);
            if (awq) v = h2f(f2h(v / h2f(awq[k])));
            as[m * K + k] = v;
        }
#ifdef _OPENMP
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
#endif
    {
        float *wd = (float *)malloc(sizeof(float) * K);
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
        for (size_t n = 0; n < N; n++) {
            for (size_t k = 0; k < K; k++) {
                size_t pi = n * ng + k / gs;
                wd[k] = h2f(f2h((read_q(qd, n * K + k, bits) - h2f(zeros[pi])) * h2f(scales[pi])));
            }
            for (size_t m = 0; m < M; m++) {
                float acc = 0.0f;
                for (size_t k = 0; k < K; k++) acc += as[m * K + k] * wd[k];
                c[m * N + n] = f2h(acc);
            }
        }
        free(wd);
    }
    free(as);
}

static inline float dot_row(const uint8_t *qd, const uint16_t *scales, const uint16_t *zeros,
                            const float *xs, size_t n, size_t K, size_t gs, int bits) {
    const size_t ng = (K + gs - 1) / gs;
    float acc = 0.0f;
    for (size_t k = 0; k < K; k++) {
        size_t pi = n * ng + k / gs;
        float w = (read_q(qd, n * K + k, bits) - h2f(zeros[pi])) * h2f(scales[pi]);
        acc += xs[k] * w;
    }
    return acc;
}

/* Fused FFN: out[n] = f16( silu(gate.x) * (up.x) ), silu(g) = g / (1 + expf(-g)), dots kept in f32.
 * crates/ironmill-inference/src/metal/shaders/quantized/affine_fused.metal:9-108
 * gate and up each [I,K] with their own scales/zeros; one shared awq vector. */
EXPORT void orc_ffn_gate_up_act(const uint8_t *gq, const uint16_t *gs_, const uint16_t *gz,
                                const uint8_t *uq, const uint16_t *us_, const uint16_t *uz,
                                const uint16_t *awq, const uint16_t *x, uint16_t *out,
                                size_t I, size_t K, size_t gsz, int bits, size_t B, int threads) {
    (void)threads;
    float *xs = (float *)malloc(sizeof(float) * B * K);
    for (size_t b = 0; b < B; b++)
        for (size_t k = 0; k < K; k++) {
            float v = h2f(x[b * K + k]);
            if (awq) v = v / h2f(awq[k]);
            xs[b * K + k] = v;
        }
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for (size_t n = 0; n < I; n++)
        for (size_t b = 0; b < B; b++) {
            float g = dot_row(gq, gs_, gz, xs + b * K, n, K, gsz, bits);
            float u = dot_row(uq, us_, uz, xs + b * K, n, K, gsz, bits);
            float act = g / (1.0f + expf(-g));
            out[b * I + n] = f2h(act * u);
        }
    free(xs);
}

/* Fused residual + RMSNorm + matvec.
 * crates/ironmill-inference/src/metal/shaders/norm/superblock_fused_norm.metal:21-124
 * r = f32(a)+f32(b); ss = sum r^2; rms_inv = 1/sqrt(ss/K + eps);
 * y[n] = f16(rms_inv * sum_k (r_k*gamma_k [/awq_k]) * w[n,k]);
 * residual_out = f16(r); normed_out = f16(r * rms_inv * gamma).  One token per row of a/b. */
EXPORT void orc_fused_residual_norm_matvec(const uint16_t *a, const uint16_t *b, const uint16_t *gamma,
                                           const uint8_t *qd, const uint16_t *scales, const uint16_t *zeros,
                                           const uint16_t *awq, float eps,
                                           uint16_t *y, uint16_t *residual_out, uint16_t *normed_out,
                                           size_t N, size_t K, size_t gs, int bits, size_t B, int threads) {
    (void)threads;
    for (size_t t = 0; t < B; t++) {
        float *xs = (float *)malloc(sizeof(float) * K);
        float ss = 0.0f;
        for (size_t k = 0; k < K; k++) {
            float r = h2f(a[t * K + k]) + h2f(b[t * K + k]);
            ss += r * r;
            float nv = r * h2f(gamma[k]);
            if (awq) nv = nv / h2f(awq[k]);
            xs[k] = nv;
        }
        float rms_inv = 1.0f / sqrtf(ss / (float)K + eps);
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
        for (size_t n = 0; n < N; n++)
            y[t * N + n] = f2h(dot_row(qd, scales, zeros, xs, n, K, gs, bits) * rms_inv);
        for (size_t k = 0; k < K; k++) {
            float r = h2f(a[t * K + k]) + h2f(b[t * K + k]);
            if (residual_out) residual_out[t * K + k] = f2h(r);
            if (normed_out) normed_out[t * K + k] = f2h(r * rms_inv * h2f(gamma[k]));
        }
        free(xs);
    }
}

/* Dense fp16 matvec (lm_head): y = f16(sum_k f32(W[n,k]) f32(x[k])), logical row-major W.
 * crates/ironmill-inference/src/metal/shaders/linear/matvec.metal:30-84 */
EXPORT void orc_matvec_f16(const uint16_t *w, const uint16_t *x, uint16_t *y,
                           size_t N, size_t K, size_t B, int threads) {
    (void)threads;
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for (size_t n = 0; n < N; n++)
        for (size_t b = 0; b < B; b++) {
            float acc = 0.0f;
            for (size_t k = 0; k < K; k++) acc += h2f(w[n * K + k]) * h2f(x[b * K + k]);
            y[b * N + n] = f2h(acc);
        }
}

/* ------------------------------------------------------------------------
 * Norms, embedding, RoPE
 * ---------------------------------------------------------------------- */

/* crates/ironmill-inference/src/metal/shaders/norm/normalization.metal:19-57 */
EXPORT void orc_rms_norm(const uint16_t *x, const uint16_t *gamma, uint16_t *out,
                         size_t H, size_t T, float eps) {
    for (size_t t = 0; t < T; t++) {
        float ss = 0.0f;
        for (size_t i = 0; i < H; i++) { float v = h2f(x[t * H + i]); ss += v * v; }
        float rms_inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (size_t i = 0; i < H; i++)
            out[t * H + i] = f2h(h2f(x[t * H + i]) * rms_inv * h2f(gamma[i]));
    }
}

/* crates/ironmill-inference/src/metal/shaders/norm/fused_residual_norm.metal:33-75:
 * residual = f16(a+b); normed from the unrounded f32 sum. */
EXPORT void orc_fused_residual_rms_norm(const uint16_t *a, const uint16_t *b, const uint16_t *gamma,
                                        uint16_t *normed, uint16_t *residual,
                                        size_t H, size_t T, float eps) {
    for (size_t t = 0; t < T; t++) {
        float ss = 0.0f;
        for (size_t i = 0; i < H; i++) {
            float v = h2f(a[t * H + i]) + h2f(b[t * H + i]);
            residual[t * H + i] = f2h(v);
            ss += v * v;
        }
        float rms_inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (size_t i = 0; i < H; i++) {
            float v = h2f(a[t * H + i]) + h2f(b[t * H + i]);
            normed[t * H + i] = f2h(v * rms_inv * h2f(gamma[i]));
        }
    }
}

/* crates/ironmill-inference/src/metal/shaders/elementwise/elementwise.metal:14-23 */
EXPORT void orc_residual_add(const uint16_t *a, const uint16_t *b, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = f2h(h2f(a[i]) + h2f(b[i]));
}

/* crates/ironmill-inference/src/metal/shaders/norm/fused_embedding_norm.metal:29-72:
 * gather fp16 row * embed_scale (zeros when token >= vocab) -> raw; RMSNorm*gamma -> normed. */
EXPORT void orc_embedding_norm(const uint32_t *tokens, const uint16_t *table, const uint16_t *gamma,
                               uint16_t *normed, uint16_t *raw, size_t H, size_t T, size_t vocab,
                               float eps, float embed_scale) {
    for (size_t t = 0; t < T; t++) {
        uint32_t tok = tokens[t];
        int valid = tok < vocab;
        float ss = 0.0f;
        for (size_t i = 0; i < H; i++) {
            float v = valid ? h2f(table[(size_t)tok * H + i]) * embed_scale : 0.0f;
            raw[t * H + i] = f2h(v);
            ss += v * v;
        }
        float rms_inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (size_t i = 0; i < H; i++) {
            float v = valid ? h2f(table[(size_t)tok * H + i]) * embed_scale : 0.0f;
            normed[t * H + i] = f2h(v * rms_inv * h2f(gamma[i]));
        }
    }
}

/* crates/ironmill-core/src/rope.rs:22-49 (precompute_rope_cache): f64 math, direct f64->f16. */
EXPORT void orc_rope_table(size_t head_dim, size_t max_pos, double theta, size_t rotary_dim,
                           uint16_t *cos_out, uint16_t *sin_out) {
    size_t half = head_dim / 2, rd = rotary_dim ? rotary_dim : head_dim, rh = rd / 2;
    for (size_t p = 0; p < max_pos; p++)
        for (size_t i = 0; i < half; i++) {
            if (i < rh) {
                double freq = 1.0 / pow(theta, 2.0 * (double)i / (double)rd);
                double ang = (double)p * freq;
                cos_out[p * half + i] = d2h(cos(ang));
                sin_out[p * half + i] = d2h(sin(ang));
            } else {
                cos_out[p * half + i] = d2h(1.0);
                sin_out[p * half + i] = d2h(0.0);
            }
        }
}

/* crates/ironmill-inference/src/metal/shaders/rope/rope.metal:21-60: half-split pairs (d, d+hd/2),
 * in place on qk [T, heads, hd]; position = seq_offset + t. */
EXPORT void orc_rope(uint16_t *qk, const uint16_t *cosc, const uint16_t *sinc,
                     size_t heads, size_t hd, size_t seq_offset, size_t T) {
    size_t half = hd / 2;
    for (size_t t = 0; t < T; t++)
        for (size_t h = 0; h < heads; h++)
            for (size_t d = 0; d < half; d++) {
                size_t ci = (seq_offset + t) * half + d;
                float c = h2f(cosc[ci]), s = h2f(sinc[ci]);
                size_t base = (t * heads + h) * hd;
                float x0 = h2f(qk[base + d]), x1 = h2f(qk[base + d + half]);
                qk[base + d] = f2h(x0 * c - x1 * s);
                qk[base + d + half] = f2h(x0 * s + x1 * c);
            }
}

/* crates/ironmill-inference/src/metal/shaders/norm/fused_qk_norm_rope.metal:43-124:
 * per head RMSNorm over head_dim with [hd] weight, then half-split RoPE over the first
 * rotary_dim dims (pairs (d, d+rotary_dim/2)), remaining dims normalised only. */
EXPORT void orc_qk_norm_rope(uint16_t *q, uint16_t *k, const uint16_t *qw, const uint16_t *kw,
                             const uint16_t *cosc, const uint16_t *sinc,
                             size_t nh, size_t nkv, size_t hd, size_t rotary_dim,
                             size_t seq_offset, size_t T, float eps) {
    size_t half_rot = rotary_dim / 2, half_dim = hd / 2;
    for (size_t t = 0; t < T; t++)
        for (size_t slot = 0; slot < nh + nkv; slot++) {
            int is_q = slot < nh;
            size_t h = is_q ? slot : slot - nh, heads = is_q ? nh : nkv;
            uint16_t *p = (is_q ? q : k) + (t * heads + h) * hd;
            const uint16_t *w = is_q ? qw : kw;
            float ss = 0.0f;
            for (size_t d = 0; d < hd; d++) { float v = h2f(p[d]); ss += v * v; }
            float rms_inv = 1.0f / sqrtf(ss / (float)hd + eps);
            size_t pos = seq_offset + t;
            for (size_t d = 0; d < half_rot; d++) {
                float lo = h2f(p[d]) * rms_inv * h2f(w[d]);
                float hi = h2f(p[d + half_rot]) * rms_inv * h2f(w[d + half_rot]);
                float c = h2f(cosc[pos * half_dim + d]), s = h2f(sinc[pos * half_dim + d]);
                p[d] = f2h(lo * c - hi * s);
                p[d + half_rot] = f2h(lo * s + hi * c);
            }
            for (size_t d = rotary_dim; d < hd; d++)
                p[d] = f2h(h2f(p[d]) * rms_inv * h2f(w[d]));
        }
}

/* ------------------------------------------------------------------------
 * TurboQuant constants
 * crates/ironmill-inference/src/turboquant/codebook.rs:20-200
 * ---------------------------------------------------------------------- */

static double horner(const double *c, int n, double x) {
    double r = c[0];
    for (int i = 1; i < n; i++) r = r * x + c[i];
    return r;
}

/* codebook.rs:187-200: erf, Abramowitz & Stegun 7.1.26-style 5-term form as written there. */
static double orc_erf(double x) {
    static const double a[5] = {1.061405429, -1.453152027, 1.421413741, -0.284496736, 0.254829592};
    const double p = 0.3275911;
    double sign = x < 0.0 ? -1.0 : 1.0;
    x = fabs(x);
    double t = 1.0 / (1.0 + p * x);
    /* (((((a5 t + a4) t) + a3) t + a2) t + a1) t */
    double poly = ((((a[0] * t + a[1]) * t + a[2]) * t + a[3]) * t + a[4]) * t;
    double y = 1.0 - poly * exp(-x * x);
    return sign * y;
}
static double normal_pdf(double x) { return exp(-0.5 * x * x) / sqrt(2.0 * M_PI); }
static double normal_cdf(double x) { return 0.5 * (1.0 + orc_erf(x * M_SQRT1_2)); }

/* codebook.rs:114-184: Beasley-Springer-Moro inverse normal CDF with the coefficient
 * values that file uses (some are shortened there; parity needs the same digits). */
static double normal_quantile(double p) {
    if (p <= 0.0) return -INFINITY;
    if (p >= 1.0) return INFINITY;
    double t = p - 0.5;
    if (fabs(t) <= 0.42) {
        static const double nc[4] = {2.5066282746310002, 18.6150006252966, 41.39119773534996, 25.44106049637689};
        static const double dc[5] = {14.382029373388, 63.690613, 84.681, 40.304, 1.0};
        double r = t * t;
        return t * horner(nc, 4, r) / horner(dc, 5, r);
    }
    double r = t < 0.0 ? p : 1.0 - p;
    double s = sqrt(-log(r));
    double res;
    if (s <= 5.0) {
        static const double nc[8] = {0.000124818987, 0.0227061845, 0.2728688, 1.3058437,
                                     2.7580128, 2.2311569, 0.6462025, 0.001612};
        static const double dc[8] = {0.000038746, 0.00745102, 0.09234118, 0.4710441,
                                     1.0507501, 1.0, 0.2127601, 1.0};
        double ss = s - 1.6;
        res = horner(nc, 8, ss) / horner(dc, 8, ss);
    } else {
        static const double nc[8] = {0.0000000271, 0.00000342556, 0.000170717, 0.004531901,
                                     0.06871337, 0.56419917, 1.9715909, 2.1538256};
        static const double dc[8] = {0.0000000393, 0.00000489649, 0.000230147, 0.005492439,
                                     0.06353648, 0.3445453, 0.73741429, 1.0};
        double ss = s - 5.0;
        res = horner(nc, 8, ss) / horner(dc, 8, ss);
    }
    return t < 0.0 ? -res : res;
}

/* codebook.rs:84-104 (conditional_mean_gaussian). */
static double cond_mean(double sigma, double lo, double hi) {
    double lo_z = lo / sigma, hi_z = hi / sigma;
    double prob = normal_cdf(hi_z) - normal_cdf(lo_z);
    if (prob < 1e-30) {
        if (isinf(lo)) return hi;
        if (isinf(hi)) return lo;
        return (lo + hi) / 2.0;
    }
    return sigma * (normal_pdf(lo_z) - normal_pdf(hi_z)) / prob;
}

/* codebook.rs:20-52 (lloyd_max_gaussian): levels[2^bits], boundaries[2^bits-1], cast to f32. */
EXPORT void orc_lloyd_max_gaussian(size_t dim, int n_bits, float *levels_out, float *bounds_out) {
    double sigma = 1.0 / sqrt((double)dim);
    size_t n = (size_t)1 << n_bits;
    double *lv = (double *)malloc(sizeof(double) * n);
    double *nl = (double *)malloc(sizeof(double) * n);
    double *bd = (double *)malloc(sizeof(double) * n);
    for (size_t i = 0; i < n; i++) lv[i] = sigma * normal_quantile(((double)i + 0.5) / (double)n);
    for (int it = 0; it < 200; it++) {
        for (size_t i = 0; i + 1 < n; i++) bd[i] = (lv[i] + lv[i + 1]) / 2.0;
        double maxd = 0.0;
        for (size_t i = 0; i < n; i++) {
            double lo = i == 0 ? -INFINITY : bd[i - 1];
            double hi = i == n - 1 ? INFINITY : bd[i];
            nl[i] = cond_mean(sigma, lo, hi);
            double d = fabs(lv[i] - nl[i]);
            if (d > maxd) maxd = d;   /* fold(0.0, f64::max) */
        }
        memcpy(lv, nl, sizeof(double) * n);
        if (maxd < 1e-10) break;
    }
    for (size_t i = 0; i + 1 < n; i++) bounds_out[i] = (float)((lv[i] + lv[i + 1]) / 2.0);
    for (size_t i = 0; i < n; i++) levels_out[i] = (float)lv[i];
    free(lv); free(nl); free(bd);
}

/* ------------------------------------------------------------------------
 * TurboQuant encode (bit-exact gate) and decode attention
 * ---------------------------------------------------------------------- */

/* crates/ironmill-inference/src/shaders/turboquant_helpers.metal:128-157
 * (hadamard_rotate_inplace): x *= sign; unnormalised WHT butterfly steps 1,2,..,hd/2;
 * x *= (sign * (1/sqrt(hd))) with the product formed first. */
static void hadamard_rotate(float *x, const float *signs, size_t hd) {
    for (size_t d = 0; d < hd; d++) x[d] = x[d] * signs[d];
    for (size_t step = 1; step < hd; step *= 2)
        for (size_t i = 0; i < hd / 2; i++) {
            size_t j = (i / step) * (step * 2) + (i % step);
            float a = x[j], b = x[j + step];
            x[j] = a + b;
            x[j + step] = a - b;
        }
    float scale = 1.0f / sqrtf((float)hd);
    for (size_t d = 0; d < hd; d++) x[d] = x[d] * (signs[d] * scale);
}
EXPORT void orc_hadamard_rotate(float *x, const float *signs, size_t hd) { hadamard_rotate(x, signs, hd); }

/* Threadgroup tree reduction with hd threads, one element per thread:
 * r[t] += r[t+s] for s = hd/2, hd/4, .., 1 (turboquant.metal:101-109). */
static float tree_sum(float *r, size_t hd) {
    for (size_t s = hd / 2; s > 0; s >>= 1)
        for (size_t t = 0; t < s; t++) r[t] = r[t] + r[t + s];
    return r[0];
}

/* crates/ironmill-inference/src/metal/shaders/turboquant/turboquant.metal:52-170
 * (turboquant_cache_write) with the packing of src/shaders/turboquant_helpers.metal:24-77.
 * kv [T, nkv, hd] fp16.  cache [nkv, max_seq, hd * n_bits / 8] u8, scale_buf / r_norms [nkv, max_seq] f32.
 * n_bits = 8: one byte per element, n_levels = 128 (K: 7-bit index | QJL sign in bit 7) or 256 (V).
 * n_bits = 4: two elements per byte (element 2i in the low nibble, 2i + 1 in the high one), n_levels = 8
 * (K: 3-bit index | QJL sign in bit 3) or 16 (V).  hd must be a power of two. */
EXPORT void orc_tq_encode(const uint16_t *kv, const float *signs, const float *codebook,
                          const float *boundaries, const float *qjl, int is_k, int n_bits,
                          uint8_t *cache, float *scale_buf, float *r_norms,
                          size_t nkv, size_t hd, size_t max_seq, size_t base_pos, size_t T) {
    size_t n_levels = is_k ? ((size_t)1 << (n_bits - 1)) : ((size_t)1 << n_bits);
    size_t nb = n_levels - 1;
    /* one (token, head) per iteration, independent of the others (tokens of one call land on different positions:
     * T <= max_seq is the caller's business, as in the reference's dispatch) */
#pragma omp parallel
    {
    float *x = (float *)malloc(sizeof(float) * hd);
    float *red = (float *)malloc(sizeof(float) * hd);
    float *res = (float *)malloc(sizeof(float) * hd);
    uint8_t *qv = (uint8_t *)malloc(hd);
#pragma omp for collapse(2) schedule(static)
    for (size_t t = 0; t < T; t++)
        for (size_t h = 0; h < nkv; h++) {
            size_t pos = (base_pos + t) % max_seq;
            const uint16_t *in = kv + (t * nkv + h) * hd;
            for (size_t d = 0; d < hd; d++) x[d] = h2f(in[d]);
            hadamard_rotate(x, signs, hd);
            for (size_t d = 0; d < hd; d++) red[d] = x[d] * x[d];
            float norm = sqrtf(fmaxf(tree_sum(red, hd), 1e-20f));
            scale_buf[h * max_seq + pos] = norm;
            float inv = 1.0f / fmaxf(norm, 1e-10f);
            for (size_t d = 0; d < hd; d++) {
                float u = x[d] * inv;
                unsigned idx = 0;
                for (size_t b = 0; b < nb; b++)
                    if (u >= boundaries[b]) idx = (unsigned)b + 1;
                qv[d] = (uint8_t)idx;
            }
            if (is_k) {
                for (size_t d = 0; d < hd; d++) res[d] = x[d] * inv - codebook[qv[d]];
                for (size_t d = 0; d < hd; d++) red[d] = res[d] * res[d];
                float rn = sqrtf(fmaxf(tree_sum(red, hd), 1e-20f));
                r_norms[h * max_seq + pos] = rn;
                uint8_t sign_mask = (uint8_t)(1u << (n_bits - 1));
                for (size_t d = 0; d < hd; d++) {
                    float proj = 0.0f;
                    for (size_t k = 0; k < hd; k++) proj = proj + qjl[d * hd + k] * res[k];
                    if (proj >= 0.0f) qv[d] |= sign_mask;
                }
            }
            if (n_bits == 4) {   /* write_packed_elements, turboquant_helpers.metal:61-77 */
                uint8_t *dst = cache + (h * max_seq + pos) * (hd / 2);
                for (size_t d = 0; d < hd; d += 2) dst[d / 2] = (uint8_t)((qv[d] & 0xF) | ((d + 1 < hd ? qv[d + 1] & 0xF : 0) << 4));
            } else {
                memcpy(cache + (h * max_seq + pos) * hd, qv, hd);
            }
        }
    free(x); free(red); free(res); free(qv);
    }
}

/* crates/ironmill-inference/src/metal/shaders/turboquant/turboquant.metal:202-462
 * (turboquant_attention) and .../attention/flash_decode.metal:163-215 (fused_sdpa_reduce).
 * q [T, nh, hd] fp16; out [T, nh, hd] fp16; causal length of token t = base_pos + t + 1.
 * num_splits == 0: single pass (normalise, then un-rotate).
 * num_splits  > 0: each split accumulates its range, un-rotates its unnormalised o and the
 * reduce combines (an empty split contributes (0, -inf, 0)). Online softmax over tiles of 32. */
EXPORT void orc_tq_attention(const uint16_t *q, const uint8_t *kc, const uint8_t *vc,
                             const float *signs, const float *k_scale, const float *v_scale,
                             const float *k_cb, const float *v_cb, const float *qjl,
                             const float *k_rn, float attn_scale, int n_bits,
                             uint16_t *out, size_t nh, size_t nkv, size_t hd, size_t max_seq,
                             size_t base_pos, size_t T, size_t num_splits) {
    const size_t TILE = 32;
    const size_t bpp = n_bits == 4 ? hd / 2 : hd;   /* bytes_per_pos, turboquant_helpers.metal:24-27 */
    const unsigned emask = n_bits == 4 ? 0xFu : 0xFFu, eshift = n_bits == 4 ? 4u : 0u;
#define TQ_RAW(row, d) (n_bits == 4 ? (((row)[(d) >> 1] >> (eshift * ((d) & 1))) & emask) : (row)[d])  /* read_raw_element :36-46 */
    size_t ns = num_splits ? num_splits : 1;
    uint8_t sign_mask = (uint8_t)(1u << (n_bits - 1));
    float qjl_factor = sqrtf(2.0f / 3.14159265f) / (float)hd;
    /* one (token, head) per iteration: the heads do not interact, so the threads change nothing in the results */
#pragma omp parallel
    {
    float *qr = (float *)malloc(sizeof(float) * hd);
    float *sq = (float *)malloc(sizeof(float) * hd);
    float *o = (float *)malloc(sizeof(float) * hd);
    float *po = (float *)malloc(sizeof(float) * ns * hd);
    float *pm = (float *)malloc(sizeof(float) * ns);
    float *ps = (float *)malloc(sizeof(float) * ns);
    float scores[32];
#pragma omp for collapse(2) schedule(dynamic)
    for (size_t t = 0; t < T; t++)
        for (size_t h = 0; h < nh; h++) {
            size_t seq_len = base_pos + t + 1;
            size_t kvh = h / (nh / nkv);
            const uint16_t *qp = q + (t * nh + h) * hd;
            for (size_t d = 0; d < hd; d++) qr[d] = h2f(qp[d]);
            hadamard_rotate(qr, signs, hd);
            for (size_t d = 0; d < hd; d++) {
                float proj = 0.0f;
                for (size_t k = 0; k < hd; k++) proj += qjl[d * hd + k] * qr[k];
                sq[d] = proj;
            }
            size_t chunk = num_splits ? (seq_len + num_splits - 1) / num_splits : seq_len;
            for (size_t s = 0; s < ns; s++) {
                size_t r0 = num_splits ? s * chunk : 0;
                size_t r1 = num_splits ? (r0 + chunk < seq_len ? r0 + chunk : seq_len) : seq_len;
                for (size_t d = 0; d < hd; d++) o[d] = 0.0f;
                float m = -INFINITY, sum = 0.0f;
                if (r0 >= seq_len) { /* empty split */
                    for (size_t d = 0; d < hd; d++) po[s * hd + d] = 0.0f;
                    pm[s] = -INFINITY; ps[s] = 0.0f;
                    continue;
                }
                for (size_t ts = r0; ts < r1; ts += TILE) {
                    size_t te = ts + TILE < r1 ? ts + TILE : r1, nt = te - ts;
                    float tm = -INFINITY;
                    for (size_t p = 0; p < nt; p++) {
                        size_t ap = ts + p;
                        float kd = k_scale[kvh * max_seq + ap];
                        float w = k_rn[kvh * max_seq + ap] * qjl_factor * kd;
                        const uint8_t *row = kc + (kvh * max_seq + ap) * bpp;
                        float part = 0.0f;
                        for (size_t d = 0; d < hd; d++) {
                            uint8_t raw = (uint8_t)TQ_RAW(row, d);
                            float kval = k_cb[raw & (sign_mask - 1)] * kd;
                            float sg = (raw & sign_mask) ? 1.0f : -1.0f;
                            part += qr[d] * kval + sq[d] * sg * w;
                        }
                        scores[p] = part * attn_scale;
                        if (scores[p] > tm) tm = scores[p];
                    }
                    float nm = m > tm ? m : tm;
                    float corr = expf(m - nm);
                    m = nm;
                    sum = sum * corr;
                    float tsum = 0.0f;
                    for (size_t p = 0; p < nt; p++) { scores[p] = expf(scores[p] - nm); tsum += scores[p]; }
                    sum += tsum;
                    for (size_t d = 0; d < hd; d++) o[d] *= corr;
                    for (size_t p = 0; p < nt; p++) {
                        size_t ap = ts + p;
                        float vd = v_scale[kvh * max_seq + ap];
                        const uint8_t *row = vc + (kvh * max_seq + ap) * bpp;
                        for (size_t d = 0; d < hd; d++) o[d] += scores[p] * (v_cb[TQ_RAW(row, d)] * vd);
                    }
                }
                if (num_splits) {
                    hadamard_rotate(o, signs, hd);
                    memcpy(po + s * hd, o, sizeof(float) * hd);
                    pm[s] = m; ps[s] = sum;
                } else {
                    float denom = fmaxf(sum, 1e-10f);
                    for (size_t d = 0; d < hd; d++) o[d] /= denom;
                    hadamard_rotate(o, signs, hd);
                    for (size_t d = 0; d < hd; d++) out[(t * nh + h) * hd + d] = f2h(o[d]);
                }
            }
            if (num_splits) {
                float gm = -INFINITY;
                for (size_t s = 0; s < ns; s++) if (pm[s] > gm) gm = pm[s];
                float csum = 0.0f;
                for (size_t d = 0; d < hd; d++) o[d] = 0.0f;
                for (size_t s = 0; s < ns; s++) {
                    float corr = expf(pm[s] - gm);
                    csum += ps[s] * corr;
                    for (size_t d = 0; d < hd; d++) o[d] += po[s * hd + d] * corr;
                }
                float denom = fmaxf(csum, 1e-10f);
                for (size_t d = 0; d < hd; d++) out[(t * nh + h) * hd + d] = f2h(o[d] / denom);
            }
        }
    free(qr); free(sq); free(o); free(po); free(pm); free(ps);
    }
#undef TQ_RAW
}

/* crates/ironmill-inference/src/sampling.rs:331-339 (argmax): last maximal index under
 * total ordering (max_by returns the last of equal maxima). */
EXPORT uint32_t orc_argmax(const float *logits, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; i++)
        if (!(logits[i] < logits[best])) best = i;
    return (uint32_t)best;
}

/* Attention over an fp16 (unquantized) KV cache: the reference's path with TurboQuant off.
 *   num_splits == 0: crates/ironmill-inference/src/metal/shaders/attention/fused_sdpa.metal:52-251 (fused_sdpa; the
 *                    prefill kernel attention.metal:571-750, prefill_attention_v2, is the same arithmetic): tiles of
 *                    SDPA_BC = 32 positions, f32 dot products of fp16 q and K scaled by `scale`, online softmax that
 *                    rescales only when the running maximum moves, O += w * V for w > 0, O / max(sum, 1e-10) -> fp16.
 *   num_splits  > 0: .../flash_decode.metal:25-151 (fused_sdpa_split: chunk = ceil(seq_len / num_splits), tiles of
 *                    SPLIT_BC = 8, max_hint = -inf as ops/attention_ops.rs:396-399 passes it, unnormalised partials)
 *                    and :163-215 (fused_sdpa_reduce: global max, rescale, normalise).
 * q [T, nh, hd] fp16; caches [nkv, max_seq, hd] fp16; out [T, nh, hd] fp16; token t attends to positions
 * 0 .. base_pos + t (causal, the reference's causal_limit = seq_len - token_count + q_pos + 1). */
EXPORT void orc_sdpa_f16(const uint16_t *q, const uint16_t *kc, const uint16_t *vc, float scale, uint16_t *out,
                         size_t nh, size_t nkv, size_t hd, size_t max_seq, size_t base_pos, size_t T, size_t num_splits) {
    const size_t gq = nh / nkv;
    const size_t ns = num_splits ? num_splits : 1;
    const size_t bc = num_splits ? 8 : 32;
#pragma omp parallel
    {
    float *qf = (float *)malloc(hd * sizeof(float)), *o = (float *)malloc(hd * sizeof(float));
    float *po = (float *)malloc(ns * hd * sizeof(float)), *pm = (float *)malloc(ns * sizeof(float)), *ps = (float *)malloc(ns * sizeof(float));
    float s_tile[32];
#pragma omp for collapse(2) schedule(dynamic)
    for (size_t t = 0; t < T; t++)
        for (size_t h = 0; h < nh; h++) {
            const size_t kvh = h / gq, seq_len = base_pos + t + 1;
            const uint16_t *K = kc + kvh * max_seq * hd, *V = vc + kvh * max_seq * hd;
            for (size_t d = 0; d < hd; d++) qf[d] = h2f(q[(t * nh + h) * hd + d]);
            const size_t chunk = (seq_len + ns - 1) / ns;
            for (size_t s = 0; s < ns; s++) {
                const size_t k0 = s * chunk, k1 = k0 + chunk < seq_len ? k0 + chunk : seq_len;
                float m = -INFINITY, l = 0.0f;
                for (size_t d = 0; d < hd; d++) o[d] = 0.0f;
                for (size_t p0 = k0; p0 < k1; p0 += bc) {
                    const size_t n = p0 + bc < k1 ? bc : k1 - p0;
                    float tile_max = -INFINITY;
                    for (size_t p = 0; p < n; p++) {
                        float dot = 0.0f;
                        for (size_t d = 0; d < hd; d++) dot += qf[d] * h2f(K[(p0 + p) * hd + d]);
                        s_tile[p] = dot * scale;
                        if (s_tile[p] > tile_max) tile_max = s_tile[p];
                    }
                    const float new_max = m > tile_max ? m : tile_max;
                    if (new_max > m) {
                        const float corr = expf(m - new_max);
                        l *= corr;
                        for (size_t d = 0; d < hd; d++) o[d] *= corr;
                        m = new_max;
                    }
                    float tile_sum = 0.0f;
                    for (size_t p = 0; p < n; p++) {
                        s_tile[p] = expf(s_tile[p] - m);
                        tile_sum += s_tile[p];
                    }
                    l += tile_sum;
                    for (size_t p = 0; p < n; p++)
                        if (s_tile[p] > 0.0f)
                            for (size_t d = 0; d < hd; d++) o[d] += s_tile[p] * h2f(V[(p0 + p) * hd + d]);
                }
                if (!num_splits) {
                    const float denom = fmaxf(l, 1e-10f);
                    for (size_t d = 0; d < hd; d++) out[(t * nh + h) * hd + d] = f2h(o[d] / denom);
                } else {
                    pm[s] = k0 < k1 ? m : -INFINITY;
                    ps[s] = l;
                    for (size_t d = 0; d < hd; d++) po[s * hd + d] = o[d];
                }
            }
            if (num_splits) {
                float gm = -INFINITY;
                for (size_t s = 0; s < ns; s++) if (pm[s] > gm) gm = pm[s];
                float csum = 0.0f;
                for (size_t d = 0; d < hd; d++) o[d] = 0.0f;
                for (size_t s = 0; s < ns; s++) {
                    const float corr = expf(pm[s] - gm);
                    csum += ps[s] * corr;
                    for (size_t d = 0; d < hd; d++) o[d] += po[s * hd + d] * corr;
                }
                const float denom = fmaxf(csum, 1e-10f);
                for (size_t d = 0; d < hd; d++) out[(t * nh + h) * hd + d] = f2h(o[d] / denom);
            }
        }
    free(qf); free(o); free(po); free(pm); free(ps);
    }
}
