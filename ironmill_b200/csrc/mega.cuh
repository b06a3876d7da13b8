// Parameter blocks of the whole-token decode kernel (decode_mega.cu), filled by the engine (model.cu).
#pragma once
#include "common.cuh"

namespace im {

struct MegaPhase {         // one projection of the token; 4 per layer in execution order: qkv, o, gate/up, down
    const uint8_t *tiles;  // [nblk][G] tiles of 1088 bytes (matvec_v2.cu)
    const __half *awq;     // [K] activation scales or nullptr
    const __half *x;       // input vector [K] (plain phases) or the branch output a of (a + residual) (norm phases)
    const __half *resid;   // norm phases: residual b; nullptr = plain phase
    const __half *gamma;   // norm phases: RMSNorm weight
    __half *resid_out;     // norm phases: a + b rounded to fp16 (must not alias x / resid)
    __half *y;             // outputs [N]
    int nblk, G, N;
    // norm phases: rows below split_row multiply the unrounded normalised vector and are scaled by rms_inv afterwards
    // (the reference's fused residual + norm + projection kernel: the next layer's Q rows); rows from split_row on
    // multiply norm_out, its fp16 copy (K, V, gate, up)
    int split_row;
    int gate_up;           // tile rows 0-7 gate, 8-15 up of the same 8 outputs -> SiLU(gate) * up
    // Tensor parallel (MegaParams::world > 1).  xout = 1 + mailbox index: the outputs are this rank's partial sums of
    // a row-split projection and go to slot `rank` of that mailbox on EVERY rank instead of y, each pair of outputs in
    // one 8-byte store together with a tag that names the launch and the layer.  xin = 1 + mailbox index: operand b is
    // the fp16-rounded sum of that mailbox's `world` slots here; the reader spins on the tags, so no barrier stands
    // between a row-split projection and the phase that consumes it.
    int xout, xin;
};

struct MegaLayer {
    const __half *q_norm, *k_norm;  // QK-norm weights or nullptr
    uint8_t *kc, *vc;               // this layer's TurboQuant caches [nkv, max_seq, 128]
    float *ks, *vs, *krn;
};

struct MegaParams {
    const MegaPhase *phases;  // device, 4 * L
    const MegaLayer *layers;  // device, L
    int L, nh, nkv, q_dim, kv_dim;
    const int *pos;           // device: position of the token being decoded
    const __half *qkv;        // the QKV phase's output buffer [q | k | v]
    __half *attn_out;         // [nh * 128]
    float *qrot;              // [nh, 2, 128]
    float *po, *pm, *pl;      // split partials [nh, splits] x (128 | 1 | 1)
    const __half *cosc, *sinc;
    const float *signs, *qjl_t, *k_cb, *k_bd, *v_cb, *v_bd;
    int k_levels, v_levels;
    int tq_bits;              // cache bits per element (8 or 4)
    float eps, attn_scale, qjl_factor;
    int max_seq, rotary_dim, with_qk_norm;
    int splits;               // attention items per KV head (capacity of the partial buffers)
    int nring;                // ring slots
    int u_bytes;              // shared-memory scratch shared by the phases
    int g_max;                // largest group count of any phase (sizes the activation staging area)
    int g_norm;               // group count of the norm phases (hidden / 128): where the second staging set starts
    int g_cap;                // groups the staging arrays hold: max(g_max, 2 g_norm)
    unsigned *bar;            // 7 * L arrival counters + 1 exit counter, zero between launches
    int *err;
    unsigned long long *trace;  // optional: CTA 0 stamps %globaltimer when it leaves each barrier (7L + 2 words)
    // Tagged hand-over of the o and down projections' outputs (MegaPhase::xout / xin).  Tensor parallel: every rank runs
    // this kernel on its shard, on its own GPU, in step with the others, and the mailboxes are peer memory.  One GPU:
    // world = 1, the mailboxes are local, and the only effect is that no grid barrier follows those two projections.
    int tagged;                 // 0: plain outputs and a barrier after every projection; nothing below is read
    int world, rank;
    int xH;                     // mailbox slot length in halves (the hidden size)
    uint2 *xmail[8];            // rank r's mailboxes [4][world][xH / 2] of {two fp16 outputs, tag} as mapped here (peer memory;
                                // [rank] is local); layers alternate between mailboxes 0-1 and 2-3 (o, down)
    unsigned *xepoch;           // local: launches completed so far (part of the tag)
    unsigned wait_ms;           // patience of every bounded wait; 0 = the default (400 ms, 5 s with peers)
};

// Shared-memory bytes the kernel needs for `nring` ring slots and `u_bytes` of phase scratch.
size_t mega_smem_bytes(int nring, int u_bytes);
// Phase scratch for projections of up to G_max groups (norm phases: G_norm) and GQ query heads per KV head.
int mega_u_bytes(int G_max, int G_norm, int gq);
int mega_g_cap(int G_max, int G_norm);
// Cooperative launch; IM_ERR_BOUNDS if the shapes do not fit the kernel.
int mega_launch(const MegaParams &p, const Device *dev, cudaStream_t st);

}  // namespace im
