"""Host-side mirror of the reference's backend/session interface for the CUDA backend.

`CudaInference` implements the `InferenceEngine` trait
(crates/ironmill-inference/src/engine.rs:72-114) the way `MetalInference` does
(crates/ironmill-inference/src/metal/engine.rs:122-270, loading.rs:483-518): same method names,
argument meaning and error behaviour; every method is one call into the C ABI.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from ._lib import CudaSysError, IM_DTYPE_F16, IM_DTYPE_F32, check, lib, vp
from .bundle import ModelConfig, WeightTensor


class InferenceError(RuntimeError):
    """InferenceError (crates/ironmill-inference/src/engine.rs:17-58); `kind` names the variant."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


def _wrap(fn):
    def inner(*a, **k):
        try:
            return fn(*a, **k)
        except CudaSysError as e:  # backend error converts like From<MetalError> (metal/error.rs:47-51)
            kind = {-3: "Allocation", -7: "NotLoaded", -4: "Decode"}.get(e.code, "Runtime")
            raise InferenceError(kind, e.message) from e
    return inner


@dataclass
class CudaConfig:
    """MetalConfig counterpart (crates/ironmill-inference/src/metal/config.rs:270-413)."""
    max_seq_len: int = 2048
    prefill_chunk_size: int | None = None
    enable_turboquant: bool = True
    rotation_seed: int = 42
    n_bits: int = 8
    max_batch: int = 1
    tp_world: int = 1
    tp_rank: int = 0
    device: int = 0
    # batch-1 decode schedule: "auto" (the whole-token kernel when the model fits it), "per_kernel" (graph of
    # per-projection kernels), "tagged" (whole-token kernel with tagged hand-over of the o / down outputs on one GPU)
    decode_schedule: str = "auto"
    tp_collective: str = "auto"   # "auto" (peer-memory exchange when the ranks can map each other) or "nccl"
    wait_limit_ms: int = 0        # patience of device-side bounded waits (0 = default)

    def with_max_seq_len(self, n: int) -> "CudaConfig":
        self.max_seq_len = n
        return self

    def with_turboquant(self, bits: int) -> "CudaConfig":
        self.enable_turboquant, self.n_bits = True, bits
        return self

    def without_turboquant(self) -> "CudaConfig":
        """fp16 KV cache (MetalConfig.enable_turboquant = false: kv_scatter + fused_sdpa / FlashDecoding)."""
        self.enable_turboquant = False
        return self

    def validate(self) -> None:
        if self.max_seq_len == 0:
            raise InferenceError("Runtime", "max_seq_len must be > 0")
        if self.n_bits not in (4, 8):
            raise InferenceError("Runtime", f"n_bits must be 4 or 8, got {self.n_bits}")


class _CModelConfig(C.Structure):
    _fields_ = [("num_layers", C.c_int), ("hidden_size", C.c_int), ("intermediate_size", C.c_int), ("num_heads", C.c_int),
                ("num_kv_heads", C.c_int), ("head_dim", C.c_int), ("vocab_size", C.c_int), ("max_seq_len", C.c_int),
                ("max_batch", C.c_int), ("rms_eps", C.c_float), ("attn_scale", C.c_float), ("embed_scale", C.c_float),
                ("rope_theta", C.c_double), ("rotary_dim", C.c_int), ("qk_norm", C.c_int), ("tie_word_embeddings", C.c_int),
                ("tq_bits", C.c_int), ("rotation_seed", C.c_uint64), ("tp_world", C.c_int), ("tp_rank", C.c_int),
                ("prefill_chunk_size", C.c_int), ("decode_schedule", C.c_int), ("tp_collective", C.c_int),
                ("wait_limit_ms", C.c_int)]


@dataclass
class ModelInfo:
    """ModelInfo (crates/ironmill-core/src/model_info.rs) - the fields the decode path fills."""
    architecture: str
    num_layers: int
    hidden_size: int
    vocab_size: int
    max_seq_len: int


def _argmax_last(logits: np.ndarray) -> int:
    """Greedy pick: the LAST maximal index (crates/ironmill-inference/src/sampling.rs:331-339)."""
    return int(logits.size - 1 - np.argmax(logits[::-1]))


class Logits(np.ndarray):
    """Logits newtype: f32 vector of length vocab (crates/ironmill-inference/src/types.rs:155-187)."""


class CudaInference:
    def __init__(self, config: CudaConfig | None = None):
        """MetalInference::new (metal/engine.rs:122-165): validates the config and opens the device."""
        self.config = config or CudaConfig()
        self.config.validate()
        self._dev = C.c_void_p()
        self._model = C.c_void_p()
        self._mc: ModelConfig | None = None
        try:
            check(lib().im_cuda_device_open(C.c_int(self.config.device), C.byref(self._dev)))
        except CudaSysError as e:
            raise InferenceError("Runtime", e.message) from e

    # ---- loading -----------------------------------------------------------------------------
    @_wrap
    def load_weights(self, provider, config: CudaConfig | None = None, tq_signs=None, tq_qjl=None) -> None:
        """MetalInference::load_weights (metal/loading.rs:483-499): walks the Hugging Face tensor names
        (weight_loading.rs:163-426) and hands each tensor to the backend."""
        if config is not None:
            config.validate()
            self.config = config
        if self._model:
            lib().im_cuda_model_free(self._model)
            self._model = C.c_void_p()
        mc: ModelConfig = provider.config()
        self._mc = mc
        cc = _CModelConfig(mc.num_hidden_layers, mc.hidden_size, mc.intermediate_size, mc.num_attention_heads,
                           mc.num_key_value_heads, mc.head_dim, mc.vocab_size, self.config.max_seq_len, self.config.max_batch,
                           mc.rms_norm_eps, mc.attn_scale, float(mc.extra.get("embed_scale", 0.0) or 0.0), mc.rope_theta,
                           int(mc.extra.get("rotary_dim", 0) or 0), int(mc.has_qk_norm), int(mc.tie_word_embeddings),
                           self.config.n_bits if self.config.enable_turboquant else 16, self.config.rotation_seed, self.config.tp_world,
                           self.config.tp_rank,
                           int(self.config.prefill_chunk_size or 0),
                           {"auto": 0, "per_kernel": 1, "tagged": 2}[self.config.decode_schedule],
                           {"auto": 0, "nccl": 1}[self.config.tp_collective], int(self.config.wait_limit_ms))
        check(lib().im_cuda_model_create(self._dev, C.byref(cc), C.byref(self._model)))
        if tq_signs is not None:
            s = np.ascontiguousarray(tq_signs, dtype=np.float32)
            q = np.ascontiguousarray(tq_qjl, dtype=np.float32)
            check(lib().im_cuda_model_set_tq_constants(self._model, vp(s), vp(q)))
        names = ["model.embed_tokens.weight", "model.norm.weight"]
        if provider.has_tensor("lm_head.weight"):
            names.append("lm_head.weight")
        for i in range(mc.num_hidden_layers):
            p = f"model.layers.{i}"
            names += [f"{p}.input_layernorm.weight", f"{p}.post_attention_layernorm.weight"]
            if mc.has_qk_norm:
                names += [f"{p}.self_attn.q_norm.weight", f"{p}.self_attn.k_norm.weight"]
            names += [f"{p}.self_attn.{x}_proj.weight" for x in "qkvo"] + [f"{p}.mlp.{x}_proj.weight" for x in ("gate", "up", "down")]
        for name in names:
            if not provider.has_tensor(name):
                raise InferenceError("Runtime", f"weight provider has no tensor '{name}'")
            self._load_tensor(name, provider.tensor(name))
        check(lib().im_cuda_model_finalize(self._model))

    def _load_tensor(self, name: str, t: WeightTensor) -> None:
        if not t.quantized:
            data = np.ascontiguousarray(t.data)
            if data.dtype != np.float16:
                data = data.astype(np.float16)   # dense tensors live in fp16 on the GPU (metal/weights.rs:928-953)
            check(lib().im_cuda_model_load_dense(self._model, name.encode(), vp(data), C.c_size_t(data.size)))
            return
        if len(t.shape) != 2:
            raise InferenceError("Runtime", f"{name}: quantized tensor must be 2-D, got shape {t.shape}")
        N, K = t.shape
        sc, zp = np.ascontiguousarray(t.scale), np.ascontiguousarray(t.zero_point)
        if sc.dtype != zp.dtype:
            sc, zp = sc.astype(np.float32), zp.astype(np.float32)
        pd = IM_DTYPE_F32 if sc.dtype == np.float32 else IM_DTYPE_F16
        awq = None if t.awq_scales is None else np.ascontiguousarray(t.awq_scales, dtype=np.float16)
        codes = np.ascontiguousarray(t.data, dtype=np.uint8)
        check(lib().im_cuda_model_load_affine(self._model, name.encode(), vp(codes), vp(sc), vp(zp), C.c_int(pd), vp(awq),
                                              C.c_int(N), C.c_int(K), C.c_int(t.group_size), C.c_int(t.bit_width)))

    @_wrap
    def tp_init(self, unique_id: bytes) -> None:
        """Joins the tensor-parallel group (every rank, same unique id).  NVLS is switched off unless the environment
        says otherwise: the library's NCCL traffic is set-up, the logits gather and prefill-size all-reduces."""
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        check(lib().im_cuda_model_tp_init(self._model, unique_id))

    def tp_peer_allreduce(self) -> bool:
        """True when the row-split projections are summed by the one-shot peer-memory all-reduce, False when NCCL does it."""
        return bool(self._model) and lib().im_cuda_model_tp_peer_allreduce(self._model) == 1

    def token_kernel(self) -> bool:
        """True when batch-1 decode steps run in the whole-token kernel (one cooperative launch for all layers)."""
        return bool(self._model) and lib().im_cuda_model_token_kernel(self._model) == 1

    @staticmethod
    def tp_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(lib().im_cuda_tp_unique_id(buf))
        return buf.raw

    # ---- InferenceEngine ----------------------------------------------------------------------
    def _need_model(self):
        if not self._model:
            raise InferenceError("NotLoaded", "model not loaded")

    @_wrap
    def prefill(self, tokens) -> np.ndarray:
        self._need_model()
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.empty(self._mc.vocab_size, dtype=np.float32)
        check(lib().im_cuda_model_prefill(self._model, vp(toks), C.c_int(toks.size), vp(out)))
        return out

    @_wrap
    def prefill_all_logits(self, tokens) -> np.ndarray:
        """InferenceEngine::prefill_all_logits (metal/pipeline.rs:38-70): logits [n_tokens, vocab], one row per token."""
        self._need_model()
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.empty((toks.size, self._mc.vocab_size), dtype=np.float32)
        check(lib().im_cuda_model_prefill_all_logits(self._model, vp(toks), C.c_int(toks.size), vp(out)))
        return out

    @_wrap
    def last_hidden_state(self, rows: int = 1) -> np.ndarray:
        """MetalInference::last_hidden_state (metal/pipeline.rs:198-226): the final RMSNorm output the lm_head consumed in
        the last step, fp16 widened to f32; [hidden] for rows = 1, else [rows, hidden] (one row per sequence of the step)."""
        self._need_model()
        out = np.empty((rows, self._mc.hidden_size), dtype=np.float32)
        check(lib().im_cuda_model_last_hidden_state(self._model, C.c_int(rows), vp(out)))
        return out[0] if rows == 1 else out

    def decode_step_with_hidden(self, token: int):
        """MetalInference::decode_step_with_hidden (metal/pipeline.rs:176-196): (logits, final hidden state)."""
        logits = self.decode_step(token)
        return logits, self.last_hidden_state()

    # ---- BatchInferenceEngine (engine.rs:121-131) ------------------------------------------------
    @_wrap
    def add_sequence(self, tokens) -> int:
        """Prefills the prompt into a free cache slot and returns the SequenceId.  The sequence's next token defaults to
        the greedy pick of the prompt's last logits (batch_decode_step without arguments)."""
        self._need_model()
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.empty(self._mc.vocab_size, dtype=np.float32)
        sid = C.c_int(-1)
        check(lib().im_cuda_model_seq_add(self._model, vp(toks), C.c_int(toks.size), C.byref(sid), vp(out)))
        self._next = getattr(self, "_next", {})
        self._next[sid.value] = int(_argmax_last(out))
        return sid.value

    @_wrap
    def remove_sequence(self, seq_id: int) -> None:
        self._need_model()
        check(lib().im_cuda_model_seq_remove(self._model, C.c_int(seq_id)))
        getattr(self, "_next", {}).pop(seq_id, None)

    def sequence_position(self, seq_id: int) -> int:
        return int(lib().im_cuda_model_seq_position(self._model, C.c_int(seq_id)))

    @_wrap
    def batch_decode_step(self, tokens: dict | None = None):
        """One decode step for all active sequences (or for those named in `tokens`: {SequenceId: token}); returns
        [(SequenceId, logits)].  Without `tokens` every active sequence continues greedily from its previous logits."""
        self._need_model()
        nxt = getattr(self, "_next", {})
        feed = dict(tokens) if tokens is not None else dict(nxt)
        if not feed:
            return []
        ids = np.ascontiguousarray(sorted(feed), dtype=np.int32)
        toks = np.ascontiguousarray([feed[int(i)] for i in ids], dtype=np.uint32)
        out = np.empty((ids.size, self._mc.vocab_size), dtype=np.float32)
        check(lib().im_cuda_model_batch_decode_step(self._model, vp(ids), vp(toks), C.c_int(ids.size), vp(out)))
        for i, sid in enumerate(ids):
            nxt[int(sid)] = int(_argmax_last(out[i]))
        self._next = nxt
        return [(int(sid), out[i]) for i, sid in enumerate(ids)]

    @_wrap
    def test_missing_ranks(self, n: int) -> None:
        """Host-side fault injection (tests of the error path; `decode_schedule="tagged"` on one GPU only): n = 1 makes
        the whole-token kernel wait for a rank that does not exist until its bounded wait gives up; 0 undoes it."""
        self._need_model()
        check(lib().im_cuda_model_test_missing_ranks(self._model, C.c_int(n)))

    @_wrap
    def decode_step(self, token) -> np.ndarray:
        """One token (int) -> logits [vocab]; a sequence of B tokens -> logits [B, vocab] (lockstep batch)."""
        self._need_model()
        scalar = np.isscalar(token)
        toks = np.ascontiguousarray([token] if scalar else token, dtype=np.uint32)
        out = np.empty((toks.size, self._mc.vocab_size), dtype=np.float32)
        check(lib().im_cuda_model_decode_step(self._model, vp(toks), C.c_int(toks.size), vp(out)))
        return out[0] if scalar else out

    @_wrap
    def decode_greedy(self, first_tokens, n_steps: int):
        """n_steps greedy steps kept on the device; returns (tokens [n_steps, batch], device milliseconds)."""
        self._need_model()
        toks = np.ascontiguousarray(first_tokens, dtype=np.uint32).reshape(-1)
        out = np.zeros((max(n_steps, 1), toks.size), dtype=np.uint32)
        ms = C.c_float()
        check(lib().im_cuda_model_decode_greedy(self._model, vp(toks), C.c_int(toks.size), C.c_int(n_steps), vp(out), C.byref(ms)))
        return out[:n_steps], float(ms.value)

    @_wrap
    def reset(self) -> None:
        self._need_model()
        check(lib().im_cuda_model_reset(self._model))
        self._next = {}

    def seq_pos(self) -> int:
        return int(lib().im_cuda_model_seq_pos(self._model)) if self._model else 0

    @_wrap
    def truncate_to(self, pos: int) -> None:
        self._need_model()
        check(lib().im_cuda_model_truncate(self._model, C.c_int(pos)))

    def max_seq_len(self) -> int:
        return self.config.max_seq_len

    def model_info(self) -> ModelInfo:
        self._need_model()
        mc = self._mc
        return ModelInfo(mc.architecture, mc.num_hidden_layers, mc.hidden_size, mc.vocab_size, self.config.max_seq_len)

    def memory_usage(self) -> int | None:
        return int(lib().im_cuda_model_memory_bytes(self._model)) if self._model else None

    def restore_kv(self, slices) -> bool:
        """Not supported, like the Metal backend (engine.rs:102-113): callers re-prefill."""
        return False

    def step_bytes(self, ctx: int, batch: int = 1) -> int:
        return int(lib().im_cuda_model_step_bytes(self._model, C.c_int(ctx), C.c_int(batch)))

    def step_launches(self) -> int:
        return int(lib().im_cuda_model_step_launches(self._model))

    PROFILE_CATEGORIES = ("embed", "qkv_proj", "rope", "kv_write", "attention", "o_proj", "residual_norm", "ffn_gate_up",
                          "down_proj", "collectives", "lm_head")

    @_wrap
    def profile_step(self, batch: int = 1) -> dict:
        """Per-category GPU milliseconds of one decode step (kernel_timing of the Metal backend)."""
        self._need_model()
        ms = (C.c_float * 11)()
        check(lib().im_cuda_model_profile_step(self._model, C.c_int(batch), ms, C.c_int(11)))
        return dict(zip(self.PROFILE_CATEGORIES, [float(v) for v in ms]))

    def token_kernel_profile(self, reps: int = 8):
        """(ms per launch, {phase: microseconds per layer}) of the whole-token decode kernel, or None when the model
        does not run it (batch > 1 only, tensor parallel, non-INT4 weights)."""
        self._need_model()
        ms = C.c_float()
        ph = (C.c_float * 7)()
        rc = lib().im_cuda_model_token_kernel_profile(self._model, C.c_int(reps), C.byref(ms), ph)
        if rc == -7:
            return None
        check(rc)
        names = ("qkv", "rope_cache_write", "attention", "split_reduce", "o", "gate_up", "down")
        return float(ms.value), {n: float(v) for n, v in zip(names, ph)}

    def close(self) -> None:
        if self._model:
            lib().im_cuda_model_free(self._model)
            self._model = C.c_void_p()
        if self._dev:
            lib().im_cuda_device_free(self._dev)
            self._dev = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
