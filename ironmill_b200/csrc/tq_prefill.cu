// TurboQuant attention for prefill chunks (many query tokens against one sequence's cache).
//
// turboquant_attention (crates/ironmill-inference/src/metal/shaders/turboquant/turboquant.metal:202-462) scores every
// (token, head) against the cached positions one token at a time; with T tokens in flight the cache is dequantised T
// times.  Its score is bilinear in what the cache holds,
//     s[t, h, p] = attn_scale * ks_p * ( q~[t,h] . cbK[idx_p]  +  (r_norm_p * qjl_factor) * (S q~)[t,h] . sign_p ),
//     o[t, h]    = sum_p softmax(s)[p] * vs_p * cbV[idx_p]        (in the rotated space; rotated back afterwards),
// so a chunk can dequantise the positions ONCE into fp16 rows K' = [cbK[idx] | sign] (256 wide) and V' = cbV[idx]
// (128 wide) and run a causal flash-attention pass over them on the tensor cores: fp16 operands, f32 accumulation, the
// per-position scalars ks_p, r_norm_p * qjl_factor and vs_p applied to the f32 scores / to the fp16 weights exactly
// where the decode kernel (tq_attention_tc_kernel) applies them.  The unnormalised outputs and (max, sum) leave in the
// split-partial format with one split, and tq_reduce_kernel normalises and rotates back as for every other path.
//
// Kernel shape: a CTA owns 16 consecutive tokens of one KV head = 16 * GQ score rows, one warp per 16 rows
// (mma.sync m16n8k16).  Position tiles of 32 rows of K' / V' travel by 16-byte cp.async into padded shared-memory rows
// (528 / 272 bytes: ldmatrix meets no bank conflict), two tiles in flight.
#include "common.cuh"
#include "tq_device.cuh"

namespace im {

namespace {

constexpr int kPfTok = 16;    // tokens per CTA
constexpr int kPfN = 32;      // positions per tile
constexpr int kKRowB = 528;   // bytes of a K' row in shared memory (256 halves + 16 bytes of padding)
constexpr int kVRowB = 272;   // V' row (128 halves + padding)

// Cache rows [0, npos) of one slot -> K' [nkv][npos][256] and V' [nkv][npos][128] fp16.  One thread per 8 elements.
template <int BITS>
__global__ void tq_dequant_rows_kernel(const uint8_t *__restrict__ kc, const uint8_t *__restrict__ vc, const float *__restrict__ k_cb,
                                       const float *__restrict__ v_cb, __half *__restrict__ kd, __half *__restrict__ vd, int slot, int nkv,
                                       int max_seq, int npos) {
    pdl_trigger();
    pdl_wait();
    constexpr int kRowB = BITS == 4 ? kHd / 2 : kHd;
    constexpr unsigned kIdx = (1u << (BITS - 1)) - 1u, kSign = 1u << (BITS - 1), kAll = (1u << BITS) - 1u;
    const int c = threadIdx.x & 15;                       // chunk of 8 elements
    const int pos = blockIdx.x * 16 + (threadIdx.x >> 4);
    const int kvh = blockIdx.y;
    if (pos >= npos) return;
    const size_t row = ((size_t)slot * nkv + kvh) * max_seq + pos;
    unsigned kb[8], vb[8];
    if (BITS == 8) {
        const uint2 kw = *reinterpret_cast<const uint2 *>(kc + row * kRowB + 8 * c), vw = *reinterpret_cast<const uint2 *>(vc + row * kRowB + 8 * c);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            kb[i] = ((i < 4 ? kw.x : kw.y) >> (8 * (i & 3))) & 255u;
            vb[i] = ((i < 4 ? vw.x : vw.y) >> (8 * (i & 3))) & 255u;
        }
    } else {
        const unsigned kw = *reinterpret_cast<const unsigned *>(kc + row * kRowB + 4 * c), vw = *reinterpret_cast<const unsigned *>(vc + row * kRowB + 4 * c);
#pragma unroll
        for (int i = 0; i < 8; i++) {  // element 2j in the low nibble of byte j
            kb[i] = (kw >> (4 * i)) & 15u;
            vb[i] = (vw >> (4 * i)) & 15u;
        }
    }
    __half kcv[8], ksv[8], vv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        kcv[i] = __float2half_rn(k_cb[kb[i] & kIdx]);
        ksv[i] = __float2half_rn((kb[i] & kSign) ? 1.0f : -1.0f);
        vv[i] = __float2half_rn(v_cb[vb[i] & kAll]);
    }
    const size_t orow = (size_t)kvh * npos + pos;
    *reinterpret_cast<uint4 *>(kd + orow * 256 + 8 * c) = *reinterpret_cast<const uint4 *>(kcv);
    *reinterpret_cast<uint4 *>(kd + orow * 256 + 128 + 8 * c) = *reinterpret_cast<const uint4 *>(ksv);
    *reinterpret_cast<uint4 *>(vd + orow * 128 + 8 * c) = *reinterpret_cast<const uint4 *>(vv);
}

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ unsigned pack2h(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&h);
}

struct PrefillParams {
    const float *qrot;         // [T, nh, 2, 128]: rotated query, S * rotated query (the second half is not read when qjl_t is given)
    const float *qjl_t;        // optional: the transposed QJL matrix [k][d] f32; the kernel then projects the rotated queries itself
    const __half *kd, *vd;     // [nkv][npos][256], [nkv][npos][128]
    const float *ks, *vs, *krn;  // cache side arrays [slots, nkv, max_seq]
    float *po, *pm, *pl;       // partials, one split: [T * nh] x (128 | 1 | 1)
    const int *pos_dev;        // position of the slot before this chunk
    float attn_scale, qjl_factor;
    int slot, nh, nkv, max_seq, T, npos, base_pos;
};

// grid (ceil(T / 16), nkv); block GQ warps; dynamic shared memory pf_smem_bytes(GQ).
template <int GQ>
__global__ void __launch_bounds__(GQ * 32, GQ == 8 ? 1 : 2) tq_prefill_attention_kernel(const PrefillParams p) {
    constexpr int M = kPfTok * GQ, NT = GQ * 32;
    extern __shared__ __align__(16) unsigned char pf_smem[];
    unsigned char *qs = pf_smem;                               // [M][528]: (q~ | S q~) fp16 per score row
    unsigned char *kt = qs + M * kKRowB;                       // [2][32][528]
    unsigned char *vt = kt + 2 * kPfN * kKRowB;                // [2][32][272]
    float *sc = reinterpret_cast<float *>(vt + 2 * kPfN * kVRowB);  // [2][3][32]: ks, r_norm * qjl_factor, vs of the tile's positions
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int tb = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y;  // the latest tokens attend to the most positions: longest CTAs first
    pdl_trigger();
    pdl_wait();
    const int P = p.base_pos + (p.pos_dev ? p.pos_dev[p.slot] : 0);
    // queries of this block's rows: row r = (token r / GQ, head r % GQ); rows of tokens past T stay zero
    for (int i = tid; i < M * 32; i += NT) {
        const int r = i >> 5, c8 = i & 31;  // 8 values per item
        const int tok = tb * kPfTok + r / GQ, h = kvh * GQ + r % GQ;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p.qjl_t && c8 >= 16) continue;  // S q~ is computed below
        if (tok < p.T) {
            const float *src = p.qrot + ((size_t)tok * p.nh + h) * 256 + 8 * c8;
            const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
            v = make_uint4(pack2h(a.x, a.y), pack2h(a.z, a.w), pack2h(b.x, b.y), pack2h(b.z, b.w));
        }
        *reinterpret_cast<uint4 *>(qs + r * kKRowB + 16 * c8) = v;
    }
    // positions this block needs: 0 .. P + (last token of the block), inside what was dequantised
    const int last_tok = min(tb * kPfTok + kPfTok - 1, p.T - 1);
    const int n_end = min(P + last_tok + 1, p.npos);
    const int ntiles = (n_end + kPfN - 1) / kPfN;
    const size_t side = ((size_t)p.slot * p.nkv + kvh) * p.max_seq;
    const __half *kd = p.kd + (size_t)kvh * p.npos * 256, *vd = p.vd + (size_t)kvh * p.npos * 128;
    auto load_tile = [&](int buf, int tile) {
        const int p0 = tile * kPfN;
        for (int i = tid; i < kPfN * 32; i += NT) {  // K': 32 chunks of 16 bytes per row
            const int r = i >> 5, c = i & 31;
            const int pos = min(p0 + r, n_end - 1);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(kt + (buf * kPfN + r) * kKRowB + 16 * c)),
                         "l"(kd + (size_t)pos * 256 + 8 * c)
                         : "memory");
        }
        for (int i = tid; i < kPfN * 16; i += NT) {  // V': 16 chunks per row
            const int r = i >> 4, c = i & 15;
            const int pos = min(p0 + r, n_end - 1);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(vt + (buf * kPfN + r) * kVRowB + 16 * c)),
                         "l"(vd + (size_t)pos * 128 + 8 * c)
                         : "memory");
        }
        if (tid < kPfN) {
            const int pos = min(p0 + tid, n_end - 1);
            sc[(buf * 3 + 0) * kPfN + tid] = p.ks[side + pos];
            sc[(buf * 3 + 1) * kPfN + tid] = p.krn[side + pos] * p.qjl_factor;
            sc[(buf * 3 + 2) * kPfN + tid] = p.vs[side + pos];
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const unsigned qs_a = (unsigned)__cvta_generic_to_shared(qs + (warp * 16 + (lane & 15)) * kKRowB + (lane >> 4) * 16);
    if (p.qjl_t) {
        // S q~ for this block's rows on the tensor cores: [16 rows x 128] x S^T [128 x 128] per warp, the matrix as fp16 in
        // the (still empty) tile buffers, rows of 272 bytes.  The per-(token, head) launch that otherwise does this reads
        // the 64 KB matrix from L2 once per row: a sixth of a 2048-token prefill.  fp16 operands like every other product
        // of this kernel; the result is rounded to fp16 as the score products read it.
        unsigned char *stm = kt;  // 128 rows x 272 bytes <= the K' and V' tile buffers together
        for (int i = tid; i < kHd * 16; i += NT) {
            const int k = i >> 4, c = i & 15;
            const float4 a = *reinterpret_cast<const float4 *>(p.qjl_t + k * kHd + 8 * c), b = *reinterpret_cast<const float4 *>(p.qjl_t + k * kHd + 8 * c + 4);
            *reinterpret_cast<uint4 *>(stm + k * kVRowB + 16 * c) = make_uint4(pack2h(a.x, a.y), pack2h(a.z, a.w), pack2h(b.x, b.y), pack2h(b.z, b.w));
        }
        __syncthreads();
        const unsigned st_a = (unsigned)__cvta_generic_to_shared(stm + (lane & 15) * kVRowB + (lane >> 4) * 16);
#pragma unroll 1
        for (int nd = 0; nd < 16; nd += 2) {
            float c0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                unsigned a[4], b[4];
                ldsm_x4(a, qs_a + kk * 32);
                ldsm_x4_t(b, st_a + kk * 16 * kVRowB + nd * 16);
                mma16816(c0, a[0], a[1], a[2], a[3], b[0], b[1]);
                mma16816(c1, a[0], a[1], a[2], a[3], b[2], b[3]);
            }
            unsigned char *r0p = qs + (warp * 16 + g) * kKRowB + 256 + (8 * nd + 2 * t) * 2, *r1p = r0p + 8 * kKRowB;
            *reinterpret_cast<unsigned *>(r0p) = pack2h(c0[0], c0[1]);
            *reinterpret_cast<unsigned *>(r1p) = pack2h(c0[2], c0[3]);
            *reinterpret_cast<unsigned *>(r0p + 16) = pack2h(c1[0], c1[1]);
            *reinterpret_cast<unsigned *>(r1p + 16) = pack2h(c1[2], c1[3]);
        }
        __syncthreads();  // the matrix is no longer needed: the tile copies may overwrite it
    }
    // this thread's two score rows: g and g + 8 of the warp's 16
    const int row0 = warp * 16 + g, row1 = row0 + 8;
    const int tok0 = tb * kPfTok + row0 / GQ, tok1 = tb * kPfTok + row1 / GQ;
    const int lim0 = tok0 < p.T ? P + tok0 : -1, lim1 = tok1 < p.T ? P + tok1 : -1;  // last position the row attends to
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    if (ntiles > 0) load_tile(0, 0);
    for (int it = 0; it < ntiles; it++) {
        const int buf = it & 1, p0 = it * kPfN;
        if (it + 1 < ntiles) {
            load_tile(buf ^ 1, it + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        // ---- scores: centroid part (dims 0-127 of K') and sign part (128-255), 4 blocks of 8 positions ----
        float sc_c[4][4], sc_s[4][4];
#pragma unroll
        for (int nb = 0; nb < 4; nb++)
#pragma unroll
            for (int e = 0; e < 4; e++) sc_c[nb][e] = sc_s[nb][e] = 0.0f;
        // ldmatrix rows of K': lanes 0-7 / 8-15: positions l & 7 at dims k0 / k0 + 8; lanes 16-31 the next 8 positions
        const unsigned kt_a = (unsigned)__cvta_generic_to_shared(kt + (buf * kPfN + (lane & 7) + 8 * (lane >> 4)) * kKRowB + ((lane >> 3) & 1) * 16);
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            unsigned a[4], b01[4], b23[4];
            ldsm_x4(a, qs_a + kk * 32);
            ldsm_x4(b01, kt_a + kk * 32);                   // positions 0-15 of the tile
            ldsm_x4(b23, kt_a + 16 * kKRowB + kk * 32);     // positions 16-31
            if (kk < 8) {
                mma16816(sc_c[0], a[0], a[1], a[2], a[3], b01[0], b01[1]);
                mma16816(sc_c[1], a[0], a[1], a[2], a[3], b01[2], b01[3]);
                mma16816(sc_c[2], a[0], a[1], a[2], a[3], b23[0], b23[1]);
                mma16816(sc_c[3], a[0], a[1], a[2], a[3], b23[2], b23[3]);
            } else {
                mma16816(sc_s[0], a[0], a[1], a[2], a[3], b01[0], b01[1]);
                mma16816(sc_s[1], a[0], a[1], a[2], a[3], b01[2], b01[3]);
                mma16816(sc_s[2], a[0], a[1], a[2], a[3], b23[0], b23[1]);
                mma16816(sc_s[3], a[0], a[1], a[2], a[3], b23[2], b23[3]);
            }
        }
        // ---- scale, mask, online softmax (rows g and g + 8; a row's 32 columns sit in the four lanes of its quad) ----
        const float *ksv = sc + (buf * 3 + 0) * kPfN, *rwv = ksv + kPfN, *vsv = rwv + kPfN;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 4; nb++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int col = 8 * nb + 2 * t + (e & 1), pos = p0 + col;
                const int lim = (e < 2) ? lim0 : lim1;
                const float s = p.attn_scale * (ksv[col] * (sc_c[nb][e] + rwv[col] * sc_s[nb][e]));
                sc_c[nb][e] = (pos <= lim && pos < n_end) ? s : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], sc_c[nb][e]);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = m_new == -INFINITY ? 1.0f : __expf(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        unsigned pa[2][4];  // A fragments of the weights (x V scale), two blocks of 16 positions
#pragma unroll
        for (int nb = 0; nb < 4; nb++) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float s = sc_c[nb][e];
                w[e] = s == -INFINITY ? 0.0f : __expf(s - m_run[e >> 1]);
                l_run[e >> 1] += w[e];
                w[e] *= vsv[8 * nb + 2 * t + (e & 1)];
            }
            pa[nb >> 1][(nb & 1) * 2 + 0] = pack2h(w[0], w[1]);  // row g,     positions 8 nb + 2t, + 1
            pa[nb >> 1][(nb & 1) * 2 + 1] = pack2h(w[2], w[3]);  // row g + 8
        }
        // ---- outputs: O[rows][dims] += W[rows][positions] V'[positions][dims] ----
        // ldmatrix.trans rows of V': lanes 0-15 positions l & 15 at dims n0, lanes 16-31 the same positions at dims n0 + 8
#pragma unroll
        for (int kb = 0; kb < 2; kb++) {
            const unsigned vt_a = (unsigned)__cvta_generic_to_shared(vt + (buf * kPfN + 16 * kb + (lane & 15)) * kVRowB + (lane >> 4) * 16);
#pragma unroll
            for (int nd = 0; nd < 16; nd += 2) {
                unsigned b[4];
                ldsm_x4_t(b, vt_a + nd * 16);
                mma16816(o[nd], pa[kb][0], pa[kb][1], pa[kb][2], pa[kb][3], b[0], b[1]);
                mma16816(o[nd + 1], pa[kb][0], pa[kb][1], pa[kb][2], pa[kb][3], b[2], b[3]);
            }
        }
        __syncthreads();  // everybody is done with this buffer before the tile after next lands in it
    }
    // ---- partials: unnormalised outputs, running max and sum (one split) ----
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        const int row = r == 0 ? row0 : row1, tok = r == 0 ? tok0 : tok1;
        if (tok < p.T) {
            const size_t hidx = (size_t)tok * p.nh + kvh * GQ + row % GQ;
#pragma unroll
            for (int nd = 0; nd < 16; nd++)
                *reinterpret_cast<float2 *>(p.po + hidx * kHd + 8 * nd + 2 * t) = make_float2(o[nd][2 * r], o[nd][2 * r + 1]);
            if (t == 0) {
                p.pm[hidx] = m_run[r];
                p.pl[hidx] = l_run[r];
            }
        }
    }
}

template <int GQ>
constexpr size_t pf_smem_bytes() {
    return (size_t)kPfTok * GQ * kKRowB + 2 * kPfN * kKRowB + 2 * kPfN * kVRowB + 2 * 3 * kPfN * sizeof(float);
}

template <int GQ>
int pf_launch(const PrefillParams &p, const Device *dev, cudaStream_t st) {
    auto kern = tq_prefill_attention_kernel<GQ>;
    static DeviceOnce once;
    if (once.first(dev->ordinal)) IM_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pf_smem_bytes<GQ>()));
    IM_CUDA_CHECK(launch_k(kern, dim3((p.T + kPfTok - 1) / kPfTok, p.nkv), dim3(GQ * 32), pf_smem_bytes<GQ>(), st, p));
    return IM_OK;
}

}  // namespace

bool tq_prefill_takes(int nh, int nkv) {
    if (nkv <= 0 || nh % nkv != 0) return false;
    const int gq = nh / nkv;
    return gq == 1 || gq == 2 || gq == 4 || gq == 8;
}

size_t tq_prefill_scratch_bytes(int nkv, int max_seq) { return (size_t)nkv * max_seq * (256 + 128) * sizeof(__half); }

// One sequence's prefill chunk: T tokens whose rows are already in the cache at positions pos_dev[slot] .. + T - 1;
// ctx_end = the host's count of cached positions after the chunk (bounds the dequantisation).  partials: T * nh * 130
// floats; dq: tq_prefill_scratch_bytes(nkv, max_seq).  IM_ERR_BOUNDS when the head grouping is not 1, 2, 4 or 8.
int tq_prefill_attention_launch(const Tq *tq, float *partials, void *dq, const float *qrot, const uint8_t *kc, const uint8_t *vc, const float *ks,
                                const float *vs, const float *krn, float attn_scale, __half *out, int slot, int nh, int nkv, int max_seq,
                                const int *pos_dev, int T, int ctx_end, cudaStream_t st, int base_pos, bool project_queries) {
    if (nkv <= 0 || nh % nkv != 0 || T <= 0) return IM_ERR_BOUNDS;
    const int gq = nh / nkv;
    if (gq != 1 && gq != 2 && gq != 4 && gq != 8) return IM_ERR_BOUNDS;
    const int npos = ctx_end < max_seq ? ctx_end : max_seq;
    __half *kd = static_cast<__half *>(dq), *vd = kd + (size_t)nkv * npos * 256;
    const dim3 dgrid((npos + 15) / 16, nkv);
    if (tq->n_bits == 4)
        IM_CUDA_CHECK(launch_k(tq_dequant_rows_kernel<4>, dgrid, dim3(256), 0, st, kc, vc, (const float *)tq->k_cb, (const float *)tq->v_cb, kd, vd, slot, nkv,
                               max_seq, npos));
    else
        IM_CUDA_CHECK(launch_k(tq_dequant_rows_kernel<8>, dgrid, dim3(256), 0, st, kc, vc, (const float *)tq->k_cb, (const float *)tq->v_cb, kd, vd, slot, nkv,
                               max_seq, npos));
    PrefillParams p{};
    p.qrot = qrot; p.qjl_t = project_queries ? tq->qjl_t : nullptr; p.kd = kd; p.vd = vd; p.ks = ks; p.vs = vs; p.krn = krn;
    const size_t rows = (size_t)T * nh;
    p.po = partials; p.pm = partials + rows * kHd; p.pl = p.pm + rows;
    p.pos_dev = pos_dev; p.attn_scale = attn_scale; p.qjl_factor = sqrtf(2.0f / 3.14159265f) / (float)tq->hd;
    p.slot = slot; p.nh = nh; p.nkv = nkv; p.max_seq = max_seq; p.T = T; p.npos = npos; p.base_pos = base_pos;
    int rc;
    switch (gq) {
    case 1: rc = pf_launch<1>(p, tq->dev, st); break;
    case 2: rc = pf_launch<2>(p, tq->dev, st); break;
    case 4: rc = pf_launch<4>(p, tq->dev, st); break;
    default: rc = pf_launch<8>(p, tq->dev, st); break;
    }
    if (rc != IM_OK) return rc;
    return tq_reduce_launch(tq, p.po, p.pm, p.pl, out, T, nh, 1, st);
}

}  // namespace im
