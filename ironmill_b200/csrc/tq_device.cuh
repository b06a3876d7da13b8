// Device-side bodies of the TurboQuant kernels, written against a "scope": a set of threads with its own
// barrier.  The stand-alone kernels run them with one CTA per work item (CtaScope); the whole-token decode
// kernel runs four items side by side in one CTA, each on a 128-thread group with a named barrier (GroupScope).
//   encode      crates/ironmill-inference/src/metal/shaders/turboquant/turboquant.metal:52-170
//   attention   .../turboquant/turboquant.metal:202-462, .../attention/flash_decode.metal:163-215
#pragma once
#include "common.cuh"

namespace im {

struct CtaScope {  // the whole CTA; d = threadIdx.x, n = blockDim.x
    int d, n;
    __device__ __forceinline__ void sync() const { __syncthreads(); }
};
struct GroupScope {  // n consecutive threads (a multiple of 32) of a larger CTA sharing hardware barrier `bar`
    int d, n, bar;
    __device__ __forceinline__ void sync() const { asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(n) : "memory"); }
};

constexpr int kTile = 32;          // positions per tile
constexpr int kAttnThreads = 128;  // 4 warps; thread d owns output dim d (hd = 128)
constexpr int kHd = 128;
constexpr int kPitchB = 132;       // bytes per tile row: 33 words -> conflict-free 32-bit reads
constexpr int kQPitch = 132;       // floats per query vector: +1 word per 32 -> conflict-free

// In-place randomized Hadamard rotation of NV vectors of length hd held in shared memory
// (x[v * pitch + d]); all threads of the scope must call it.  Plain float arithmetic.
template <int NV, class Scope>
__device__ __forceinline__ void hadamard_block(const Scope &sc, float *x, int pitch, const float *__restrict__ signs, int hd) {
    for (int i = sc.d; i < NV * hd; i += sc.n) {
        const int v = i / hd, d = i % hd;
        x[v * pitch + d] *= signs[d];
    }
    sc.sync();
    for (int step = 1; step < hd; step <<= 1) {
        for (int i = sc.d; i < NV * (hd / 2); i += sc.n) {
            const int v = i / (hd / 2), e = i % (hd / 2);
            const int j = (e / step) * (2 * step) + (e % step);
            float *p = x + v * pitch;
            const float a = p[j], b = p[j + step];
            p[j] = a + b;
            p[j + step] = a - b;
        }
        sc.sync();
    }
    const float scale = 1.0f / sqrtf((float)hd);
    for (int i = sc.d; i < NV * hd; i += sc.n) {
        const int v = i / hd, d = i % hd;
        x[v * pitch + d] *= signs[d] * scale;
    }
    sc.sync();
}

// The same rotation for ONE vector with thread d of the scope holding element d (scope size = hd >= 32): strides
// below 32 on warp shuffles, the rest through xs (hd floats).  Same pairs and operations as hadamard_block.
template <class Scope>
__device__ __forceinline__ float hadamard_thread(const Scope &sc, float v, float sg, float *xs, int hd) {
    const int d = sc.d;
    v *= sg;
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, step);
        v = (d & step) ? o - v : v + o;
    }
    for (int step = 32; step < hd; step <<= 1) {
        xs[d] = v;
        sc.sync();
        const float o = xs[d ^ step];
        v = (d & step) ? o - v : v + o;
        sc.sync();
    }
    return v * (sg * (1.0f / sqrtf((float)hd)));
}

// ---------------------------------------------------------------- encode (bit-exact)
struct EncodeTables {
    const float *signs, *cb, *bounds, *qjl_t;  // bounds = suffix minima; qjl_t = transposed QJL matrix [k][d]
    int n_levels, is_k;
    int bits;  // cache bits per element: 8 (one byte each) or 4 (element 2i in the low nibble of byte i, 2i + 1 in the high one)
};
// bytes of one cached position (bytes_per_pos, crates/ironmill-inference/src/shaders/turboquant_helpers.metal:24-27)
__host__ __device__ __forceinline__ int tq_row_bytes(int bits, int hd) { return bits == 4 ? hd / 2 : hd; }

// The QJL projection of a 128-vector held in shared memory: thread d computes sum_k S^T[k][d] * vec[k], walking k
// upwards.  `Direct` reads the thread's matrix column itself, 64 values in flight at a time; begin() may be called
// early so that the first half travels while the caller still reduces.  EXACT selects the encoder's arithmetic
// (separate multiply and add, bit-exact with turboquant_cache_write); otherwise fused multiply-adds.
struct QjlDirect {
    const float *qjl_t;
    float sv[64];
    __device__ __forceinline__ void begin(int d, int hd) {
#pragma unroll
        for (int j = 0; j < 64; j++) sv[j] = j < hd ? qjl_t[(size_t)j * hd + d] : 0.0f;
    }
    template <bool EXACT, class Scope>
    __device__ __forceinline__ float finish(const Scope &, const float *vec, int d, int hd) {
        float proj = 0.0f;
        for (int k0 = 0; k0 < hd; k0 += 64) {
            if (k0 > 0) {
#pragma unroll
                for (int j = 0; j < 64; j++) sv[j] = k0 + j < hd ? qjl_t[(size_t)(k0 + j) * hd + d] : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 64; j++)
                if (k0 + j < hd) proj = EXACT ? __fadd_rn(proj, __fmul_rn(sv[j], vec[k0 + j])) : fmaf(sv[j], vec[k0 + j], proj);
        }
        return proj;
    }
};

// Encodes one head vector; thread d of the scope (n = hd threads) holds element d (already widened from
// fp16).  sh = 3*hd floats.  Every operation and its order follow turboquant_cache_write; the QJL dot
// product walks k upwards with separate multiply and add, reading the transposed matrix so that the
// warp's loads coalesce.
// Sum of the scope's hd values in the order of the reference's shared-memory tree (stride hd/2, hd/4, ... 1:
// r[d] += r[d + s] for d < s), with the strides below 32 done by warp shuffles: lane d < s adds the value of lane
// d + s, which is exactly r[d + s] of the tree.  buf: hd floats; every thread gets the total.  hd >= 32.
template <class Scope>
__device__ __forceinline__ float tq_tree_sum(const Scope &sc, float v, float *buf, int hd) {
    const int d = sc.d;
    buf[d] = v;
    sc.sync();
    const int l = d & 31;
    // strides >= 32 straight from shared memory, in the tree's order: width w -> w/2 ... until 32 values remain
    // r_w[j] = r_2w[j] + r_2w[j + w]; evaluated recursively for j = lane
    float r;
    if (hd == 128) {
        r = __fadd_rn(__fadd_rn(buf[l], buf[l + 64]), __fadd_rn(buf[l + 32], buf[l + 96]));
    } else {
        // generic: fold the top halves down one stride at a time (every warp repeats the same reads)
        for (int s = hd / 2; s >= 32; s >>= 1) {
            float t = 0.0f;
            if (d < s) t = __fadd_rn(buf[d], buf[d + s]);
            sc.sync();
            if (d < s) buf[d] = t;
            sc.sync();
        }
        r = buf[l];
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) r = __fadd_rn(r, __shfl_down_sync(0xffffffffu, r, s));
    r = __shfl_sync(0xffffffffu, r, 0);
    sc.sync();  // buf may be rewritten by the caller
    return r;
}

// Encodes one head vector; thread d of the scope (n = hd threads) holds element d (already widened from
// fp16).  sh = 3*hd floats.  Every operation follows turboquant_cache_write: the same butterfly pairs with the
// same add / subtract, the same summation trees, the QJL dot product walking k upwards with separate multiply and
// add (reading the transposed matrix so that the warp's loads coalesce).  Butterfly strides below 32 and the
// tails of the trees run on warp shuffles instead of shared memory + barriers; the operands are the same.
template <class Scope, class Proj>
__device__ __forceinline__ void tq_encode_body(const Scope &sc, float xin, const EncodeTables &tb, float *sh, int hd, uint8_t *cache_row,
                                               float *scale_out, float *rnorm_out, float sg, Proj &pj) {
    float *xs = sh, *red = sh + hd, *res = sh + 2 * hd;
    const int d = sc.d;
    float v = __fmul_rn(xin, sg);
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {  // pair (j, j + step): lower index gets a + b, upper a - b
        const float o = __shfl_xor_sync(0xffffffffu, v, step);
        v = (d & step) ? __fsub_rn(o, v) : __fadd_rn(v, o);
    }
    for (int step = 32; step < hd; step <<= 1) {
        xs[d] = v;
        sc.sync();
        const float o = xs[d ^ step];
        v = (d & step) ? __fsub_rn(o, v) : __fadd_rn(v, o);
        sc.sync();
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    const float x = __fmul_rn(v, __fmul_rn(sg, scale));
    const float ss = tq_tree_sum(sc, __fmul_rn(x, x), red, hd);
    const float norm = __fsqrt_rn(fmaxf(ss, 1e-20f));
    if (d == 0) *scale_out = norm;
    const float inv = __fdiv_rn(1.0f, fmaxf(norm, 1e-10f));
    const float u = __fmul_rn(x, inv);
    // The reference scans all boundaries and keeps the LAST b with u >= boundaries[b]
    // (index b + 1).  Its 7- and 8-bit tables are not monotone, so that is not a plain
    // upper bound; `bounds` holds the suffix minima of the table, which are monotone and
    // give the same answer: max{b : boundaries[b] <= u} = max{b : min(boundaries[b..]) <= u}.
    int lo = 0, hi = tb.n_levels - 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (u >= tb.bounds[mid]) lo = mid + 1; else hi = mid;
    }
    unsigned byte = (unsigned)lo;
    if (tb.is_k) {
        const float r = __fsub_rn(u, tb.cb[lo]);
        res[d] = r;
        pj.begin(d, hd);  // a direct projector's first loads travel while the residual norm is reduced
        const float rs = tq_tree_sum(sc, __fmul_rn(r, r), red, hd);  // its barriers also publish res[]
        if (d == 0) *rnorm_out = __fsqrt_rn(fmaxf(rs, 1e-20f));
        const float proj = pj.template finish<true>(sc, res, d, hd);
        if (proj >= 0.0f) byte |= 1u << (tb.bits - 1);  // the QJL sign rides in the top bit of the storage unit
    }
    if (tb.bits == 4) {  // write_packed_elements (turboquant_helpers.metal:61-77): even thread writes the pair
        const unsigned hi = __shfl_down_sync(0xffffffffu, byte, 1);
        if (!(d & 1)) cache_row[d >> 1] = (uint8_t)((byte & 0xFu) | ((hi & 0xFu) << 4));
    } else {
        cache_row[d] = (uint8_t)byte;
    }
    sc.sync();  // sh may be reused by the caller
}

template <class Scope>
__device__ __forceinline__ void tq_encode_body(const Scope &sc, float xin, const EncodeTables &tb, float *sh, int hd, uint8_t *cache_row,
                                               float *scale_out, float *rnorm_out, float sg) {
    QjlDirect pj{tb.qjl_t};
    tq_encode_body(sc, xin, tb, sh, hd, cache_row, scale_out, rnorm_out, sg, pj);
}
template <class Scope>
__device__ __forceinline__ void tq_encode_body(const Scope &sc, float xin, const EncodeTables &tb, float *sh, int hd, uint8_t *cache_row,
                                               float *scale_out, float *rnorm_out) {
    tq_encode_body(sc, xin, tb, sh, hd, cache_row, scale_out, rnorm_out, tb.signs[sc.d]);
}

// ---------------------------------------------------------------- attention
struct AttnParams {
    const __half *q;         // [nseq*T, nh, hd]
    const uint8_t *kc, *vc;  // [nseq, nkv, max_seq, hd]
    const float *ks, *vs, *krn;  // [nseq, nkv, max_seq]
    const float *signs, *qjl, *k_cb, *v_cb;  // qjl: TRANSPOSED matrix [k][d]
    const float *qrot;       // optional [nseq*T, nh, 2, hd]: rotated query and S * rotated query, computed upstream
    float *po, *pm, *pl;     // partials [nseq*T, nh, splits] x (hd | 1 | 1)
    float attn_scale, qjl_factor;
    int nh, nkv, max_seq, base_pos, T, splits;
    const int *pos_dev;      // optional per-slot positions (added to base_pos)
    const int *slot_map;     // optional: sequence index of this launch -> cache slot (nullptr: identity)
    int bits;                // cache bits per element (8 or 4); rows hold tq_row_bytes(bits, hd) bytes
};
// Eight 4-bit elements of a cache word -> two words of one byte per element (the 8-bit layout the score and value
// loops read).  K: the 3-bit index stays in bits 0-2, the QJL sign moves from bit 3 to bit 7; V: the byte is the index.
__device__ __forceinline__ unsigned tq_spread4(unsigned x) {  // nibbles 0-3 of x (low 16 bits) -> bytes
    x &= 0xFFFFu;
    x = (x | (x << 8)) & 0x00FF00FFu;
    return (x | (x << 4)) & 0x0F0F0F0Fu;
}
__device__ __forceinline__ unsigned tq_k_byte(unsigned b) { return (b & 0x07070707u) | ((b & 0x08080808u) << 4); }
__device__ __forceinline__ int cache_slot(const int *slot_map, int seq) { return slot_map ? slot_map[seq] : seq; }

__device__ __forceinline__ int qidx(int d) { return d + (d >> 5); }
template <int GQ>
__device__ __forceinline__ int qrow(int d) { return d * 2 * GQ + (d >> 4) * 4; }  // first float of dimension d's row in AttnSmem::qv

template <int GQ>
struct AttnSmem {  // per work item (128 threads)
    // queries, one row of 2 GQ floats per dimension: the GQ rotated queries, then the GQ values of S * q, so that the
    // score loop fetches all of a dimension's operands with one or two vector loads; 4 floats of padding after
    // every 16 rows keep the eight dimension slices a warp reads at once on different banks
    float qv[2 * GQ * kHd + 32];
    alignas(16) uint8_t tile[kTile * kPitchB];  // the K codes of a tile, then the V codes of the same positions
    float t_ks[kTile], t_rw[kTile], t_vs[kTile];
    float sc[GQ * kTile];
    float s_m[GQ], s_l[GQ], s_corr[GQ];
};

// Ask L2 for the first tile of an item (rows of positions below `limit` only) without holding anything in registers:
// issued before the barrier that publishes the query rotation and the new cache row, it turns the item's first cache
// reads from HBM misses into L2 hits.
__device__ __forceinline__ void tq_attention_l2_prefetch(int tid, const AttnParams &p, int kvh, int seq, int r0, int r1, int limit) {
    const size_t head_base = ((size_t)cache_slot(p.slot_map, seq) * p.nkv + kvh) * p.max_seq;
    const int nt = min(kTile, min(r1, limit) - r0);
    const size_t rowb = (size_t)tq_row_bytes(p.bits, kHd);
    if (tid < nt) {  // one row of K and of V per thread (a 128-byte line holds one 8-bit row or two 4-bit rows)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.kc + (head_base + r0 + tid) * rowb));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.vc + (head_base + r0 + tid) * rowb));
    } else if (tid >= 32 && tid < 35 && nt > 0) {  // the tile's scales: 32 floats = one line each
        const float *b = tid == 32 ? p.ks : (tid == 33 ? p.krn : p.vs);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(b + head_base + r0));
    }
}

// One (kv head, token, split) item on a 128-thread scope: positions [r0, r1) of the sequence against the GQ
// query heads of the group.  cbk / cbv: the K (128) and V (256) codebooks in shared memory, filled by the caller.
template <int GQ, class Scope>
__device__ __forceinline__ void tq_attention_item(const Scope &sc, AttnSmem<GQ> &sm, const float *cbk, const float *cbv, const AttnParams &p,
                                                  int kvh, int st, int split, int r0, int r1) {
    const int tid = sc.d, lane = tid & 31, warp = tid >> 5;
    const int seq = st / p.T;
    const int h0 = kvh * GQ;

    if (r0 >= r1) {  // empty split: neutral partial
        for (int g = 0; g < GQ; g++) {
            const size_t pi = ((size_t)st * p.nh + h0 + g) * p.splits + split;
            p.po[pi * kHd + tid] = 0.0f;
            if (tid == 0) {
                p.pm[pi] = -INFINITY;
                p.pl[pi] = 0.0f;
            }
        }
        return;
    }

    // The K / V rows of a tile travel through registers: the first tile is requested before the queries are set
    // up, each further tile while its predecessor is being scored, so the cache latency overlaps other work.
    const size_t head_base = ((size_t)cache_slot(p.slot_map, seq) * p.nkv + kvh) * p.max_seq;
    const int pr = tid >> 2, part = tid & 3;  // loader: 32 rows x 128 bytes, 32 bytes per thread
    uint4 nk0, nk1, nv0, nv1;
    float n_ks = 0.0f, n_rw = 0.0f, n_vs = 0.0f;
    auto fetch = [&](int ts) {
        const int nt = min(kTile, r1 - ts);
        nk0 = nk1 = nv0 = nv1 = make_uint4(0, 0, 0, 0);
        if (pr < nt) {
            if (p.bits == 4) {  // 64-byte rows: 16 bytes (32 elements) per thread, spread to bytes when stored
                nk0 = ldg_stream_v4(reinterpret_cast<const uint4 *>(p.kc + (head_base + ts + pr) * (kHd / 2) + part * 16));
                nv0 = ldg_stream_v4(reinterpret_cast<const uint4 *>(p.vc + (head_base + ts + pr) * (kHd / 2) + part * 16));
            } else {
                const uint4 *ksrc = reinterpret_cast<const uint4 *>(p.kc + (head_base + ts + pr) * kHd + part * 32);
                const uint4 *vsrc = reinterpret_cast<const uint4 *>(p.vc + (head_base + ts + pr) * kHd + part * 32);
                nk0 = ldg_stream_v4(ksrc);
                nk1 = ldg_stream_v4(ksrc + 1);
                nv0 = ldg_stream_v4(vsrc);
                nv1 = ldg_stream_v4(vsrc + 1);
            }
        }
        if (tid < kTile) {
            const bool ok = tid < nt;
            n_ks = ok ? p.ks[head_base + ts + tid] : 0.0f;
            n_rw = ok ? p.krn[head_base + ts + tid] * p.qjl_factor : 0.0f;
            n_vs = ok ? p.vs[head_base + ts + tid] : 0.0f;
        }
    };
    fetch(r0);

    if (tid < GQ) {
        sm.s_m[tid] = -INFINITY;
        sm.s_l[tid] = 0.0f;
    }
    if (p.qrot) {
#pragma unroll
        for (int g = 0; g < GQ; g++) {
            const float *src = p.qrot + ((size_t)st * p.nh + h0 + g) * 2 * kHd;
            sm.qv[qrow<GQ>(tid) + g] = src[tid];
            sm.qv[qrow<GQ>(tid) + GQ + g] = src[kHd + tid];
        }
    } else {
        float *qr = sm.qv;  // scratch in the old one-vector-per-head layout, converted below
#pragma unroll
        for (int g = 0; g < GQ; g++) qr[g * kQPitch + tid] = __half2float(p.q[((size_t)st * p.nh + h0 + g) * kHd + tid]);
        sc.sync();
        hadamard_block<GQ>(sc, qr, kQPitch, p.signs, kHd);
        float acc[GQ], tmp[GQ];
#pragma unroll
        for (int g = 0; g < GQ; g++) acc[g] = 0.0f;
        for (int k = 0; k < kHd; k++) {  // transposed matrix: the warp reads consecutive floats
            const float sv = p.qjl[(size_t)k * kHd + tid];
#pragma unroll
            for (int g = 0; g < GQ; g++) acc[g] = fmaf(sv, qr[g * kQPitch + k], acc[g]);
        }
#pragma unroll
        for (int g = 0; g < GQ; g++) tmp[g] = qr[g * kQPitch + tid];
        sc.sync();
#pragma unroll
        for (int g = 0; g < GQ; g++) {
            sm.qv[qrow<GQ>(tid) + g] = tmp[g];
            sm.qv[qrow<GQ>(tid) + GQ + g] = acc[g];
        }
    }
    sc.sync();

    float o[GQ];
#pragma unroll
    for (int g = 0; g < GQ; g++) o[g] = 0.0f;

    uint32_t *td = reinterpret_cast<uint32_t *>(sm.tile + pr * kPitchB + part * 32);
    for (int ts = r0; ts < r1; ts += kTile) {
        const int nt = min(kTile, r1 - ts);
        // ---- K goes to the tile buffer now, V waits in registers until the scores are done ----
        const uint4 v0 = nv0, v1 = nv1;
        if (p.bits == 4) {
            td[0] = tq_k_byte(tq_spread4(nk0.x)); td[1] = tq_k_byte(tq_spread4(nk0.x >> 16));
            td[2] = tq_k_byte(tq_spread4(nk0.y)); td[3] = tq_k_byte(tq_spread4(nk0.y >> 16));
            td[4] = tq_k_byte(tq_spread4(nk0.z)); td[5] = tq_k_byte(tq_spread4(nk0.z >> 16));
            td[6] = tq_k_byte(tq_spread4(nk0.w)); td[7] = tq_k_byte(tq_spread4(nk0.w >> 16));
        } else {
            td[0] = nk0.x; td[1] = nk0.y; td[2] = nk0.z; td[3] = nk0.w; td[4] = nk1.x; td[5] = nk1.y; td[6] = nk1.z; td[7] = nk1.w;
        }
        if (tid < kTile) {
            sm.t_ks[tid] = n_ks;
            sm.t_rw[tid] = n_rw;
            sm.t_vs[tid] = n_vs;
        }
        if (ts + kTile < r1) fetch(ts + kTile);
        sc.sync();

        // ---- scores: warp w owns positions 8w..8w+7; a lane scores TWO positions over a slice of 16 dimensions, so
        // every query row it fetches (the loop's dominant shared-memory traffic) serves both ----
        constexpr int GP = GQ < 4 ? GQ : 4;  // heads per pass: eight heads at once would not fit the register budget
#pragma unroll 1
        for (int gb = 0; gb < GQ; gb += GP) {
            const int ds = lane & 7, p0 = warp * 8 + (lane >> 3) * 2;
            float s0[GP], s1[GP], t0[GP], t1[GP];  // centroid and sign sums of the two positions
#pragma unroll
            for (int g = 0; g < GP; g++) s0[g] = s1[g] = t0[g] = t1[g] = 0.0f;
            const uint32_t *kr0 = reinterpret_cast<const uint32_t *>(sm.tile + p0 * kPitchB + ds * 16);
            const uint32_t *kr1 = reinterpret_cast<const uint32_t *>(sm.tile + (p0 + 1) * kPitchB + ds * 16);
#pragma unroll
            for (int jw = 0; jw < 4; jw++) {
                const uint32_t w0 = kr0[jw], w1 = kr1[jw];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t b0 = (w0 >> (8 * e)) & 0xffu, b1 = (w1 >> (8 * e)) & 0xffu;
                    const float kc0 = cbk[b0 & 0x7fu], kc1 = cbk[b1 & 0x7fu];
                    const float sg0 = (b0 & 0x80u) ? 1.0f : -1.0f, sg1 = (b1 & 0x80u) ? 1.0f : -1.0f;
                    float qa[GP], qb[GP];  // this dimension's row: the rotated queries and S * q of the pass's heads (vector loads)
                    {
                        const float *row = sm.qv + qrow<GQ>(ds * 16 + jw * 4 + e);
                        if (GQ == 1) {
                            const float2 v = *reinterpret_cast<const float2 *>(row);
                            qa[0] = v.x; qb[0] = v.y;
                        } else if (GQ == 2) {
                            const float4 v = *reinterpret_cast<const float4 *>(row);
                            qa[0] = v.x; qa[1] = v.y; qb[0] = v.z; qb[1] = v.w;
                        } else {
                            const float4 va = *reinterpret_cast<const float4 *>(row + gb);
                            const float4 vb = *reinterpret_cast<const float4 *>(row + GQ + gb);
                            qa[0] = va.x; qa[1] = va.y; qa[2] = va.z; qa[3] = va.w;
                            qb[0] = vb.x; qb[1] = vb.y; qb[2] = vb.z; qb[3] = vb.w;
                        }
                    }
#pragma unroll
                    for (int g = 0; g < GP; g++) {
                        s0[g] = fmaf(qa[g], kc0, s0[g]);
                        t0[g] = fmaf(qb[g], sg0, t0[g]);
                        s1[g] = fmaf(qa[g], kc1, s1[g]);
                        t1[g] = fmaf(qb[g], sg1, t1[g]);
                    }
                }
            }
            const float rw0 = sm.t_rw[p0], rw1 = sm.t_rw[p0 + 1];
#pragma unroll
            for (int g = 0; g < GP; g++) {  // the residual weight is per position: fold before the slices are summed
                s0[g] = fmaf(rw0, t0[g], s0[g]);
                s1[g] = fmaf(rw1, t1[g], s1[g]);
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    s0[g] += __shfl_xor_sync(0xffffffffu, s0[g], o);
                    s1[g] += __shfl_xor_sync(0xffffffffu, s1[g], o);
                }
            }
            if (ds == 0) {
                const float k0 = p.attn_scale * sm.t_ks[p0], k1 = p.attn_scale * sm.t_ks[p0 + 1];
#pragma unroll
                for (int g = 0; g < GP; g++) {
                    sm.sc[p0 * GQ + gb + g] = p0 < nt ? k0 * s0[g] : -INFINITY;
                    sm.sc[(p0 + 1) * GQ + gb + g] = p0 + 1 < nt ? k1 * s1[g] : -INFINITY;
                }
            }
        }
        sc.sync();

        // ---- the V codes replace the K codes; online softmax: one warp per query head, lane = position ----
        if (p.bits == 4) {
            td[0] = tq_spread4(v0.x); td[1] = tq_spread4(v0.x >> 16); td[2] = tq_spread4(v0.y); td[3] = tq_spread4(v0.y >> 16);
            td[4] = tq_spread4(v0.z); td[5] = tq_spread4(v0.z >> 16); td[6] = tq_spread4(v0.w); td[7] = tq_spread4(v0.w >> 16);
        } else {
            td[0] = v0.x; td[1] = v0.y; td[2] = v0.z; td[3] = v0.w; td[4] = v1.x; td[5] = v1.y; td[6] = v1.z; td[7] = v1.w;
        }
        for (int g = warp; g < GQ; g += kAttnThreads / 32) {
            const float s = sm.sc[lane * GQ + g];
            const float tm = warp_max(s);
            const float m_old = sm.s_m[g];
            const float m_new = fmaxf(m_old, tm);
            const float w = lane < nt ? __expf(s - m_new) : 0.0f;
            const float tsum = warp_sum(w);
            sm.sc[lane * GQ + g] = w * sm.t_vs[lane];
            if (lane == 0) {
                const float corr = __expf(m_old - m_new);
                sm.s_corr[g] = corr;
                sm.s_m[g] = m_new;
                sm.s_l[g] = sm.s_l[g] * corr + tsum;
            }
        }
        sc.sync();

        // ---- weighted V: thread d accumulates output dim d for every head of the group ----
#pragma unroll
        for (int g = 0; g < GQ; g++) o[g] *= sm.s_corr[g];
        for (int pp = 0; pp < nt; pp++) {
            const float v = cbv[sm.tile[pp * kPitchB + tid]];
#pragma unroll
            for (int g = 0; g < GQ; g++) o[g] = fmaf(sm.sc[pp * GQ + g], v, o[g]);
        }
        sc.sync();
    }

#pragma unroll
    for (int g = 0; g < GQ; g++) {
        const size_t pi = ((size_t)st * p.nh + h0 + g) * p.splits + split;
        p.po[pi * kHd + tid] = o[g];
        if (tid == 0) {
            p.pm[pi] = sm.s_m[g];
            p.pl[pi] = sm.s_l[g];
        }
    }
    sc.sync();  // sm may be reused by the caller's next item
}

// ---------------------------------------------------------------- (QK-norm +) RoPE + cache write + query rotation
//   query heads : (RMSNorm,) RoPE as fused_qk_norm_rope / rope, rounded to fp16 like the reference's q buffer,
//                 then the rotation R q and S (R q) that every attention item of the head would otherwise redo
//   key heads   : (RMSNorm,) RoPE, rounded to fp16, then the bit-exact cache write
//   value heads : the bit-exact cache write
struct PrepArgs {
    const __half *qkv;  // [nseq*T, stride]: q | k | v of one token
    int stride, k_off, v_off;
    const __half *kv;   // nullptr, or the buffer [nseq*T, kv_stride] that holds the K and V rows (k_off / v_off index it)
    int kv_stride;
    const __half *qw, *kw, *cosc, *sinc;
    int nh, nkv, rotary_dim, with_norm, T, max_seq, base_pos;
    float eps;
    const int *pos_dev;
    const int *slot_map;  // optional: sequence index -> cache slot (positions and cache rows are per slot)
    float *qrot;    // [nseq*T, nh, 2, hd]
    __half *q_out;  // optional dense roped q [nseq*T, nh, hd]
    EncodeTables ktab, vtab;
    uint8_t *kc, *vc;
    float *ks, *vs, *krn;
    int no_q_proj;  // query heads: skip the QJL projection (its consumer computes it)
};

// One head (slot in [0, nh + 2 nkv)) of token st on a 128-thread scope.  sh: 3*128 + 4 floats.  pj: the QJL
// projector (key heads project sh + 256, query heads sh).
template <class Scope, class Proj>
__device__ __forceinline__ void tq_prep_item(const Scope &sc, const PrepArgs &a, float *sh, int slot, int st, Proj &pj) {
    float *red = sh + 3 * kHd;
    const int d = sc.d;
    const int seq = cache_slot(a.slot_map, st / a.T), t = st % a.T;  // from here on `seq` names the cache slot
    const int pos_abs = a.base_pos + (a.pos_dev ? a.pos_dev[seq] : 0) + t;
    const __half *tok = a.qkv + (size_t)st * a.stride;
    const __half *tokkv = a.kv ? a.kv + (size_t)st * a.kv_stride : tok;
    const float sg = a.ktab.signs[d];  // requested together with the head's values, not after the RoPE
    if (slot >= a.nh + a.nkv) {  // value head
        const int h = slot - a.nh - a.nkv;
        const size_t row = ((size_t)seq * a.nkv + h) * a.max_seq + pos_abs % a.max_seq;
        tq_encode_body(sc, __half2float(tokkv[a.v_off + h * kHd + d]), a.vtab, sh, kHd, a.vc + row * tq_row_bytes(a.vtab.bits, kHd), a.vs + row, (float *)nullptr, sg);
        return;
    }
    const bool is_q = slot < a.nh;
    const int h = is_q ? slot : slot - a.nh;
    const __half *src = (is_q ? tok : tokkv + a.k_off) + h * kHd;
    const __half *w = is_q ? a.qw : a.kw;
    float x = __half2float(src[d]);
    // the rotation's table entries are requested with the head's values, not after the norm's barrier
    const int half_rot = a.rotary_dim / 2;
    const int ri = d < half_rot ? d : d - half_rot;
    float rc = 1.0f, rs = 0.0f;
    if (d < a.rotary_dim) {
        rc = __half2float(a.cosc[(size_t)pos_abs * (kHd / 2) + ri]);
        rs = __half2float(a.sinc[(size_t)pos_abs * (kHd / 2) + ri]);
    }
    if (a.with_norm) {
        float ss = warp_sum(x * x);
        if ((d & 31) == 0) red[d >> 5] = ss;
        sc.sync();
        const float tot = red[0] + red[1] + red[2] + red[3];
        x = x * rsqrtf(tot / (float)kHd + a.eps) * __half2float(w[d]);
    }
    sh[d] = x;
    sc.sync();
    float y = x;
    if (d < a.rotary_dim) {
        const float lo = sh[ri], hi = sh[ri + half_rot];
        y = d < half_rot ? lo * rc - hi * rs : lo * rs + hi * rc;
    }
    const __half yh = __float2half_rn(y);
    sc.sync();
    if (!is_q) {
        const size_t row = ((size_t)seq * a.nkv + h) * a.max_seq + pos_abs % a.max_seq;
        tq_encode_body(sc, __half2float(yh), a.ktab, sh, kHd, a.kc + row * tq_row_bytes(a.ktab.bits, kHd), a.ks + row, a.krn + row, sg, pj);
        return;
    }
    if (a.q_out) a.q_out[((size_t)st * a.nh + h) * kHd + d] = yh;
    const float rq = hadamard_thread(sc, __half2float(yh), sg, sh + kHd, kHd);
    sh[d] = rq;
    float *dst = a.qrot + ((size_t)st * a.nh + h) * 2 * kHd;
    dst[d] = rq;
    sc.sync();
    if (a.no_q_proj) return;
    pj.begin(d, kHd);
    const float acc = pj.template finish<false>(sc, sh, d, kHd);
    dst[kHd + d] = acc;
    sc.sync();  // sh may be reused by the caller
}

template <class Scope>
__device__ __forceinline__ void tq_prep_item(const Scope &sc, const PrepArgs &a, float *sh, int slot, int st) {
    QjlDirect pj{a.ktab.qjl_t};
    tq_prep_item(sc, a, sh, slot, st, pj);
}

// Combine the splits of one (token, head), normalise, rotate back, write fp16.
// The inverse rotation is linear, so applying it once after the combination equals the
// reference's per-split rotation up to float rounding.  x: 128 floats of shared memory.
template <class Scope>
__device__ __forceinline__ void tq_reduce_item(const Scope &sc, float *x, const float *__restrict__ po, const float *__restrict__ pm,
                                               const float *__restrict__ pl, const float *__restrict__ signs, __half *__restrict__ out,
                                               size_t head_index, int splits_stride, int splits_used) {
    const int d = sc.d;
    const size_t base = head_index * splits_stride;
    const float sg = signs[d];
    float gm = -INFINITY;
    for (int s0 = 0; s0 < splits_used; s0 += 8) {  // eight loads in flight at a time; combined in split order
        float m[8];
#pragma unroll
        for (int j = 0; j < 8; j++) m[j] = s0 + j < splits_used ? pm[base + s0 + j] : -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; j++) gm = fmaxf(gm, m[j]);
    }
    float acc = 0.0f, lsum = 0.0f;
    for (int s0 = 0; s0 < splits_used; s0 += 8) {
        float m[8], l[8], o[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const bool live = s0 + j < splits_used;
            m[j] = live ? pm[base + s0 + j] : -INFINITY;
            l[j] = live ? pl[base + s0 + j] : 0.0f;
            o[j] = live ? po[(base + s0 + j) * kHd + d] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float corr = m[j] == -INFINITY ? 0.0f : __expf(m[j] - gm);
            lsum += l[j] * corr;
            acc += o[j] * corr;
        }
    }
    const float r = hadamard_thread(sc, acc / fmaxf(lsum, 1e-10f), sg, x, kHd);
    out[head_index * kHd + d] = __float2half_rn(r);
}

}  // namespace im
