"""CPU oracle of the whole decode step (test infrastructure): numpy glue over the oracle primitives,
following the reference's schedule and its fp16 rounding points
(crates/ironmill-inference/src/metal/pipeline.rs:424-1313; end-of-layer fusion
crates/ironmill-inference/src/metal/attention.rs:616-702).  Weights are dequantised once to f32
with w = (q - z) * s from the fp16 scale / zero point the GPU sees; dot products accumulate in f32."""
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
    def __init__(self, cfg, tensors, tqc, max_seq, flip_rate=0.0):
        """flip_rate > 0 flips the lowest fp16 bit of that fraction of the activations entering every layer:
        a stand-in for "another correct implementation" used to measure how far last-bit differences grow."""
        self.cfg, self.tq, self.max_seq = cfg, tqc, max_seq
        self.flip_rate, self._flip_rng = flip_rate, np.random.default_rng(12345)
        g = lambda n: tensors[n].data.astype(np.float16)  # noqa: E731
        self.embed = g("model.embed_tokens.weight")
        self.lm = (self.embed if cfg.tie_word_embeddings else g("lm_head.weight")).astype(np.float32)
        self.final_norm = g("model.norm.weight")
        self.L = []
        nkv, hd = cfg.num_key_value_heads, cfg.head_dim
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
            d["kc"] = np.zeros((nkv, max_seq, hd), np.uint8)
            d["vc"] = np.zeros((nkv, max_seq, hd), np.uint8)
            d["ks"], d["vs"], d["kr"] = (np.zeros((nkv, max_seq), np.float32) for _ in range(3))
            self.L.append(d)
        self.cos, self.sin = orc.rope_table(hd, max_seq, cfg.rope_theta, cfg.extra.get("rotary_dim"))
        self.pos = 0

    def _flip(self, a16):
        v = np.ascontiguousarray(a16).view(np.uint16).copy()
        v[self._flip_rng.random(v.shape) < self.flip_rate] ^= 1
        return v.view(np.float16)

    @staticmethod
    def _mv(w, awq, x16):
        x = x16.astype(np.float32)
        if awq is not None:
            x = x / awq
        return (x @ w.T).astype(np.float16)

    def forward(self, tokens):
        """tokens: T ids appended at the current position; returns f32 logits of the last one."""
        c, T = self.cfg, len(tokens)
        nh, nkv, hd, eps = c.num_attention_heads, c.num_key_value_heads, c.head_dim, np.float32(c.rms_norm_eps)
        norm_out, hidden = orc.embedding_norm(np.asarray(tokens, np.uint32), self.embed, self.L[0]["in_ln"], float(eps))
        qkv = None
        for li, d in enumerate(self.L):
            if li == 0:
                qkv = self._mv(d["qkv"], d["qkv_awq"], norm_out)
            if self.flip_rate:
                qkv, hidden = self._flip(qkv), self._flip(hidden)
            q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
            if c.has_qk_norm:
                q, k = orc.qk_norm_rope(q, k, d["qn"], d["kn"], self.cos, self.sin, nh, nkv, hd, self.pos, float(eps))
            else:
                q = orc.rope(q, self.cos, self.sin, nh, hd, self.pos)
                k = orc.rope(k, self.cos, self.sin, nkv, hd, self.pos)
            orc.tq_encode(k, self.tq, True, d["kc"], d["ks"], d["kr"], nkv, self.max_seq, self.pos)
            orc.tq_encode(np.ascontiguousarray(v), self.tq, False, d["vc"], d["vs"], None, nkv, self.max_seq, self.pos)
            attn = orc.tq_attention(q, d["kc"], d["vc"], self.tq, d["ks"], d["vs"], d["kr"], c.attn_scale, nh, nkv,
                                    self.max_seq, self.pos).reshape(T, nh * hd)
            o = self._mv(d["o"], d["o_awq"], attn)
            norm_out, residual = orc.fused_residual_rms_norm(hidden, o, d["post_ln"], float(eps))
            x = norm_out.astype(np.float32)
            if d["ffn_awq"] is not None:
                x = x / d["ffn_awq"]
            gt, up = x @ d["gate"].T, x @ d["up"].T
            act = (gt / (np.float32(1.0) + np.exp(-gt))) * up
            ffn = act.astype(np.float16)
            down = self._mv(d["down"], d["down_awq"], ffn)
            r = residual.astype(np.float32) + down.astype(np.float32)
            hidden = r.astype(np.float16)
            if li + 1 < len(self.L):
                nx = self.L[li + 1]
                rms_inv = (np.float32(1.0) / np.sqrt((r * r).sum(-1, keepdims=True, dtype=np.float32) / np.float32(r.shape[-1]) + eps)).astype(np.float32)
                gam = nx["in_ln"].astype(np.float32)
                norm_out = (r * rms_inv * gam).astype(np.float16)
                xn = r * gam
                if nx["qkv_awq"] is not None:
                    xn = xn / nx["qkv_awq"]
                qkv = ((xn @ nx["qkv"].T) * rms_inv).astype(np.float16)
        last = orc.rms_norm(hidden[-1:], self.final_norm, float(eps))
        logits = (last.astype(np.float32) @ self.lm.T).astype(np.float16).astype(np.float32)
        self.pos += T
        return logits[0]
