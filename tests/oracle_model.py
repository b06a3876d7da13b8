"""CPU oracle of the whole decode step (test infrastructure): numpy glue over the oracle primitives,
following the reference's schedule and its fp16 rounding points
(crates/ironmill-inference/src/metal/pipeline.rs:424-1313; end-of-layer fusion
crates/ironmill-inference/src/metal/attention.rs:616-702; FFN dispatch metal/ffn.rs:13-150; matvec / matmul
choice metal/ops/mod.rs LinearKernelKind::for_token_count; attention split rule metal/attention.rs:394-413).
Weights are dequantised once to f32 with w = (q - z) * s from the fp16 scale / zero point the GPU sees;
dot products accumulate in f32.

Rounding points of one token (token_count == 1, INT4 weights):
  embedding -> hidden f16, norm_out f16; layer 0: Q, K, V = matvec(norm_out f16) -> f16;
  layers >= 1: K, V = matvec(norm_out f16); Q comes from the previous layer's fused
  residual + norm + projection kernel, which multiplies the UNROUNDED f32 normalised vector;
  (QK-norm,) RoPE in place -> f16; cache write; attention (split in chunks of ceil(seq / splits) once the
  sequence holds 256 positions, each split rotating its partial back) -> f16; o -> f16;
  fused residual + norm -> residual f16, norm_out f16; gate/up read norm_out f16, their f32 dot products feed
  SiLU(g) * u -> f16; down -> f16; residual + down -> hidden f16 (+ norm_out f16, next Q).
token_count > 1 (prefill): every projection runs the matmul form f16(sum f16(x / awq) * f16((q - z) s)), gate and up
are rounded to f16 before SiLU(g) * u, no projection is fused into a norm, attention is a single pass per token.
INT8 weights never take the fused kernels (they exist for 4 bits only)."""
import numpy as np

from oracle import oracle as orc


def synth_model(cfg, seed=0, bits=4, gs=128, awq=False, gamma_jitter=0.0, threads=8):
    """Random-init tensors of the given ModelConfig: linear weights ~ N(0, 0.02) quantized by the CPU
    oracle (INT4/INT8 group `gs`, optional AWQ scales ~ U(0.5, 2) shared by projections with the same
    input), fp16 embeddings / lm_head ~ N(0, 0.02), norm weights 1 (+ optional jitter)."""
    from ironmill_b200.bundle import WeightTensor
    from tests import helpers as H
    Hd, I, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    t = {}

    def dense(name, shape, std=0.02, ones=False):
        r = H.rng_for(name, seed)
        a = (1.0 + gamma_jitter * r.standard_normal(shape)) if ones else r.standard_normal(shape) * std
        t[name] = WeightTensor(a.astype(np.float16), tuple(shape), "float16")

    def quant(name, N, K, awq_vec):
        w = (H.rng_for(name, seed).standard_normal((N, K)) * 0.02).astype(np.float16)
        codes, sc, zp = orc.quantize_groups(w, gs, bits, awq=awq_vec, threads=threads)
        packed = orc.pack_int4(codes) if bits == 4 else codes.reshape(-1).copy()
        t[name] = WeightTensor(packed, (N, K), "uint8", sc, zp, bits, gs, 1, awq_vec)

    dense("model.embed_tokens.weight", (cfg.vocab_size, Hd))
    if not cfg.tie_word_embeddings:
        dense("lm_head.weight", (cfg.vocab_size, Hd))
    dense("model.norm.weight", (Hd,), ones=True)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        dense(f"{p}.input_layernorm.weight", (Hd,), ones=True)
        dense(f"{p}.post_attention_layernorm.weight", (Hd,), ones=True)
        if cfg.has_qk_norm:
            dense(f"{p}.self_attn.q_norm.weight", (hd,), ones=True)
            dense(f"{p}.self_attn.k_norm.weight", (hd,), ones=True)
        a_in = H.make_awq(Hd, seed, f"{p}.attn_in") if awq else None
        a_o = H.make_awq(nh * hd, seed, f"{p}.o_in") if awq else None
        a_ffn = H.make_awq(Hd, seed, f"{p}.ffn_in") if awq else None
        a_dn = H.make_awq(I, seed, f"{p}.down_in") if awq else None
        quant(f"{p}.self_attn.q_proj.weight", nh * hd, Hd, a_in)
        quant(f"{p}.self_attn.k_proj.weight", nkv * hd, Hd, a_in)
        quant(f"{p}.self_attn.v_proj.weight", nkv * hd, Hd, a_in)
        quant(f"{p}.self_attn.o_proj.weight", Hd, nh * hd, a_o)
        quant(f"{p}.mlp.gate_proj.weight", I, Hd, a_ffn)
        quant(f"{p}.mlp.up_proj.weight", I, Hd, a_ffn)
        quant(f"{p}.mlp.down_proj.weight", Hd, I, a_dn)
    return t


class DictProvider:
    """WeightProvider over an in-memory dict (the MockProvider of the reference's bundle tests,
    crates/ironmill-compile/src/gpu/bundle.rs:366-395)."""

    def __init__(self, cfg, tensors):
        self._cfg, self._t = cfg, tensors

    def config(self):
        return self._cfg

    def tensor_names(self):
        return list(self._t)

    def has_tensor(self, n):
        return n in self._t

    def tensor(self, n):
        return self._t[n]


def _deq(t):
    """f32 matrix (q - z) * s with fp16-rounded params, plus the f32 AWQ divisor (or None)."""
    N, K = t.shape
    codes = orc.unpack_int4(t.data, N * K).reshape(N, K) if t.bit_width == 4 else np.asarray(t.data).reshape(N, K)
    s = orc.f32_to_f16(t.scale.astype(np.float32)).astype(np.float32) if t.scale.dtype != np.float16 else t.scale.astype(np.float32)
    z = orc.f32_to_f16(t.zero_point.astype(np.float32)).astype(np.float32) if t.zero_point.dtype != np.float16 else t.zero_point.astype(np.float32)
    G = s.shape[1]
    w = (codes.reshape(N, G, -1).astype(np.float32) - z[:, :, None]) * s[:, :, None]
    awq = None if t.awq_scales is None else t.awq_scales.astype(np.float32)
    return w.reshape(N, K), awq


class OracleModel:
    """deviations: names of departures from the reference's rounding points, used to measure what each one costs
    (every one of them is a legitimate "same arithmetic contract" choice an implementation could make):
      kv_unrounded   K and V of layers >= 1 from the unrounded normalised vector (like Q)
      ffn_unrounded  gate/up from the unrounded normalised vector
      no_split       decode attention in a single pass whatever the length (one rotation back instead of one per split)
      act_q16        projection inputs rounded to 16-bit integers per group of 128 (scale amax / 32639)
      act_q24        the same with 24-bit integers (scale amax / 8355711)
      sum_order      dot products summed as two halves of K (another f32 summation order)
      prefill_matvec prefill projections in the matvec form (no f16 rounding of x / awq and of the weights)"""

    def __init__(self, cfg, tensors, tqc, max_seq, flip_rate=0.0, deviations=(), kv_f16=False):
        """flip_rate > 0 flips the lowest fp16 bit of that fraction of the activations entering every layer:
        a stand-in for "another correct implementation" used to measure how far last-bit differences grow."""
        self.cfg, self.tq, self.max_seq = cfg, tqc, max_seq
        self.kv_f16 = kv_f16  # TurboQuant off: fp16 K / V rows in the cache (metal/attention.rs:491-612)
        self.flip_rate, self._flip_rng = flip_rate, np.random.default_rng(12345)
        self.dev = frozenset(deviations)
        unknown = self.dev - {"kv_unrounded", "ffn_unrounded", "no_split", "act_q16", "act_q24", "sum_order", "prefill_matvec"}
        assert not unknown, unknown
        g = lambda n: tensors[n].data.astype(np.float16)  # noqa: E731
        self.embed = g("model.embed_tokens.weight")
        self.lm = (self.embed if cfg.tie_word_embeddings else g("lm_head.weight")).astype(np.float32)
        self.final_norm = g("model.norm.weight")
        self.L = []
        nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.bits = tensors["model.layers.0.self_attn.q_proj.weight"].bit_width
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}"
            d = {"in_ln": g(f"{p}.input_layernorm.weight"), "post_ln": g(f"{p}.post_attention_layernorm.weight")}
            if cfg.has_qk_norm:
                d["qn"], d["kn"] = g(f"{p}.self_attn.q_norm.weight"), g(f"{p}.self_attn.k_norm.weight")
            ws = [_deq(tensors[f"{p}.self_attn.{x}_proj.weight"]) for x in "qkv"]
            d["qkv"], d["qkv_awq"] = np.concatenate([w for w, _ in ws], 0), ws[0][1]
            d["o"], d["o_awq"] = _deq(tensors[f"{p}.self_attn.o_proj.weight"])
            d["gate"], d["ffn_awq"] = _deq(tensors[f"{p}.mlp.gate_proj.weight"])
            d["up"], _ = _deq(tensors[f"{p}.mlp.up_proj.weight"])
            d["down"], d["down_awq"] = _deq(tensors[f"{p}.mlp.down_proj.weight"])
            if kv_f16:
                d["k16"], d["v16"] = np.zeros((nkv, max_seq, hd), np.float16), np.zeros((nkv, max_seq, hd), np.float16)
            else:
                d["kc"] = np.zeros((nkv, max_seq, hd * tqc.n_bits // 8), np.uint8)   # n_bits = 4: two elements per byte
                d["vc"] = np.zeros((nkv, max_seq, hd * tqc.n_bits // 8), np.uint8)
                d["ks"], d["vs"], d["kr"] = (np.zeros((nkv, max_seq), np.float32) for _ in range(3))
            self.L.append(d)
        self._w16 = {}
        self.cos, self.sin = orc.rope_table(hd, max_seq, cfg.rope_theta, cfg.extra.get("rotary_dim"))
        self.pos = 0

    def _flip(self, a16):
        v = np.ascontiguousarray(a16).view(np.uint16).copy()
        v[self._flip_rng.random(v.shape) < self.flip_rate] ^= 1
        return v.view(np.float16)

    # ---- projections ------------------------------------------------------------------------------------------
    def _round_act(self, x):
        """The act_q16 / act_q24 deviations: x [T, K] f32 -> the values a block-integer staging would multiply."""
        top = 32639.0 if "act_q16" in self.dev else 8355711.0 if "act_q24" in self.dev else None
        if top is None or x.shape[-1] % 128:
            return x
        xg = x.reshape(x.shape[0], -1, 128)
        amax = np.abs(xg).max(-1, keepdims=True)
        safe = np.where(amax > 0, amax, np.float32(1.0))
        xi = np.clip(np.rint(xg * (np.float32(top) / safe)), -top, top).astype(np.float32)
        return (xi * (safe * np.float32(1.0 / top))).reshape(x.shape).astype(np.float32)

    def _dot(self, x, w):
        if "sum_order" in self.dev:
            h = w.shape[1] // 2
            return x[:, :h] @ w[:, :h].T + x[:, h:] @ w[:, h:].T
        return x @ w.T

    def _mv32(self, w, awq, x32):
        """Matvec form on an f32 input: f32(x) / f32(awq) against f32 (q - z) s, f32 result (not yet rounded)."""
        x = x32 if awq is None else x32 / awq
        return self._dot(self._round_act(x.astype(np.float32)), w)

    def _mv(self, w, awq, x16):
        return self._mv32(w, awq, x16.astype(np.float32)).astype(np.float16)

    def _mm(self, key, w, awq, x16):
        """Matmul form (affine_matmul.metal:44-74,119-127): both operands rounded to f16, f32 accumulation."""
        if "prefill_matvec" in self.dev:
            return self._mv(w, awq, x16)
        if key not in self._w16:
            self._w16[key] = w.astype(np.float16).astype(np.float32)
        x = x16.astype(np.float32)
        if awq is not None:
            x = (x / awq).astype(np.float16).astype(np.float32)
        return self._dot(x, self._w16[key]).astype(np.float16)

    def _proj(self, li, name, w, awq, x16, decode):
        return self._mv(w, awq, x16) if decode else self._mm((li, name), w, awq, x16)

    def forward(self, tokens):
        """tokens: T ids appended at the current position; returns f32 logits of the last one."""
        c, T = self.cfg, len(tokens)
        nh, nkv, hd, eps = c.num_attention_heads, c.num_key_value_heads, c.head_dim, np.float32(c.rms_norm_eps)
        decode = T == 1
        fused = decode and self.bits == 4          # the fused kernels exist for 4-bit weights and one token only
        norm_out, hidden = orc.embedding_norm(np.asarray(tokens, np.uint32), self.embed, self.L[0]["in_ln"], float(eps))
        pre = None  # (q or qkv) computed by the previous layer's fused residual + norm + projection
        for li, d in enumerate(self.L):
            nq = nh * hd
            if pre is not None and pre.shape[1] == d["qkv"].shape[0]:
                qkv = pre
            else:
                qkv = self._proj(li, "qkv", d["qkv"], d["qkv_awq"], norm_out, decode)
                if pre is not None:
                    qkv = np.concatenate([pre, qkv[:, nq:]], 1)
            if self.flip_rate:
                qkv, hidden = self._flip(qkv), self._flip(hidden)
            q, k, v = qkv[:, :nq], qkv[:, nq:nq + nkv * hd], qkv[:, nq + nkv * hd:]
            if c.has_qk_norm:
                q, k = orc.qk_norm_rope(q, k, d["qn"], d["kn"], self.cos, self.sin, nh, nkv, hd, self.pos, float(eps))
            else:
                q = orc.rope(q, self.cos, self.sin, nh, hd, self.pos)
                k = orc.rope(k, self.cos, self.sin, nkv, hd, self.pos)
            seq = self.pos + T
            splits = 0
            if decode and seq >= 256 and "no_split" not in self.dev:
                splits = max(2, min(-(-seq // 256), 256))
            if self.kv_f16:  # kv_scatter (shaders/kv/kv_scatter.metal:20-42), then fused_sdpa / prefill_attention_v2 / the split pair
                kk = np.asarray(k, np.float16).reshape(T, nkv, hd)
                vv = np.asarray(v, np.float16).reshape(T, nkv, hd)
                for t in range(T):
                    d["k16"][:, self.pos + t] = kk[t]
                    d["v16"][:, self.pos + t] = vv[t]
                attn = orc.sdpa_f16(q, d["k16"], d["v16"], c.attn_scale, nh, nkv, hd, self.max_seq, self.pos,
                                    num_splits=splits).reshape(T, nh * hd)
            else:
                orc.tq_encode(k, self.tq, True, d["kc"], d["ks"], d["kr"], nkv, self.max_seq, self.pos)
                orc.tq_encode(np.ascontiguousarray(v), self.tq, False, d["vc"], d["vs"], None, nkv, self.max_seq, self.pos)
                attn = orc.tq_attention(q, d["kc"], d["vc"], self.tq, d["ks"], d["vs"], d["kr"], c.attn_scale, nh, nkv,
                                        self.max_seq, self.pos, num_splits=splits).reshape(T, nh * hd)
            o = self._proj(li, "o", d["o"], d["o_awq"], attn, decode)
            norm_out, residual = orc.fused_residual_rms_norm(hidden, o, d["post_ln"], float(eps))
            if fused:
                if "ffn_unrounded" in self.dev:
                    r = hidden.astype(np.float32) + o.astype(np.float32)
                    ri = (np.float32(1.0) / np.sqrt((r * r).sum(-1, keepdims=True, dtype=np.float32) / np.float32(r.shape[-1]) + eps)).astype(np.float32)
                    xg = r * d["post_ln"].astype(np.float32)
                    gt, up = self._mv32(d["gate"], d["ffn_awq"], xg) * ri, self._mv32(d["up"], d["ffn_awq"], xg) * ri
                else:
                    x = norm_out.astype(np.float32)
                    gt, up = self._mv32(d["gate"], d["ffn_awq"], x), self._mv32(d["up"], d["ffn_awq"], x)
            else:
                gt = self._proj(li, "gate", d["gate"], d["ffn_awq"], norm_out, decode).astype(np.float32)
                up = self._proj(li, "up", d["up"], d["ffn_awq"], norm_out, decode).astype(np.float32)
            ffn = ((gt / (np.float32(1.0) + np.exp(-gt))) * up).astype(np.float16)
            down = self._proj(li, "down", d["down"], d["down_awq"], ffn, decode)
            r = residual.astype(np.float32) + down.astype(np.float32)
            hidden = r.astype(np.float16)
            pre = None
            if li + 1 < len(self.L):
                nx = self.L[li + 1]
                rms_inv = (np.float32(1.0) / np.sqrt((r * r).sum(-1, keepdims=True, dtype=np.float32) / np.float32(r.shape[-1]) + eps)).astype(np.float32)
                gam = nx["in_ln"].astype(np.float32)
                norm_out = (r * rms_inv * gam).astype(np.float16)
                if fused:
                    rows = nx["qkv"].shape[0] if "kv_unrounded" in self.dev else nh * hd
                    pre = (self._mv32(nx["qkv"][:rows], nx["qkv_awq"], r * gam) * rms_inv).astype(np.float16)
        last = orc.rms_norm(hidden[-1:], self.final_norm, float(eps))
        self.last_hidden = last[0].astype(np.float32)  # norm_out after the final norm (metal/pipeline.rs:176-226)
        logits = (last.astype(np.float32) @ self.lm.T).astype(np.float16).astype(np.float32)
        self.pos += T
        return logits[0]
