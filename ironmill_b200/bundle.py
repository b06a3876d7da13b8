"""`.ironml-gpu` bundle reader and writer (the `dense` and `affine_dequantize` tensor formats).

Layout and manifest schema follow crates/ironmill-core/src/gpu/bundle.rs:34-149 (GpuBundleManifest,
TensorManifest) and the writer crates/ironmill-compile/src/gpu/bundle.rs:41-264: a directory with
`manifest.json` and `weights/<name with . and / replaced by _>.{bin,qdata,scale,zeros,awq}`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import numpy as np

_DTYPES = {"float16": np.float16, "float32": np.float32, "uint8": np.uint8, "int8": np.int8, "int32": np.int32}


class GpuBundleError(Exception):
    """GpuBundleError (crates/ironmill-core/src/gpu/bundle.rs:13-25)."""


@dataclass
class WeightTensor:
    """WeightTensor + QuantizationInfo::AffineDequantize (crates/mil-rs/src/weights.rs:520-640)."""
    data: np.ndarray                      # dense values, or packed codes (uint8) when quantized
    shape: tuple
    dtype: str = "float16"
    scale: np.ndarray | None = None       # f32 or fp16 [rows, groups]
    zero_point: np.ndarray | None = None
    bit_width: int = 0                    # 0 = dense
    group_size: int = 0
    axis: int = -1
    awq_scales: np.ndarray | None = None  # fp16 [K]

    @property
    def quantized(self) -> bool:
        return self.bit_width != 0


@dataclass
class ModelConfig:
    """ModelConfig (crates/mil-rs/src/weights.rs:57-97) restricted to the decode path's fields."""
    architecture: str = "llama"
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 128
    vocab_size: int = 0
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    extra: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        d = {k: getattr(self, k) for k in ("architecture", "hidden_size", "intermediate_size", "num_hidden_layers",
                                           "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
                                           "max_position_embeddings", "rms_norm_eps", "rope_theta", "tie_word_embeddings")}
        if self.extra:
            d["extra"] = self.extra
        return d

    @staticmethod
    def from_json(obj: dict) -> "ModelConfig":
        if not isinstance(obj, dict):
            raise GpuBundleError("model_config must be an object")
        cfg = ModelConfig()
        for k in ("architecture",):
            if not isinstance(obj.get(k), str):
                raise GpuBundleError(f"missing string field: {k}")
        for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "head_dim", "vocab_size", "max_position_embeddings"):
            if not isinstance(obj.get(k), int):
                raise GpuBundleError(f"missing integer field: {k}")
        for k in ("rms_norm_eps", "rope_theta"):
            if not isinstance(obj.get(k), (int, float)):
                raise GpuBundleError(f"missing float field: {k}")
        for k, v in obj.items():
            if k == "extra":
                cfg.extra = dict(v or {})
            elif hasattr(cfg, k):
                setattr(cfg, k, v)
        cfg.tie_word_embeddings = bool(obj.get("tie_word_embeddings", False))
        return cfg

    @property
    def has_qk_norm(self) -> bool:
        return self.architecture.lower().startswith("qwen3") or bool(self.extra.get("qk_norm"))

    @property
    def attn_scale(self) -> float:
        # crates/mil-rs/src/weights.rs:210-217: 1/sqrt(query_pre_attn_scalar) when set, else 1/sqrt(head_dim)
        q = self.extra.get("query_pre_attn_scalar")
        return float(1.0 / np.sqrt(q if q else self.head_dim))


def sanitize_tensor_name(name: str) -> str:
    return name.replace(".", "_").replace("/", "_")


def write_gpu_bundle(path: str, config: ModelConfig, tensors: dict, quantization: dict | None = None) -> None:
    """write_gpu_bundle (crates/ironmill-compile/src/gpu/bundle.rs:52-356)."""
    wdir = os.path.join(path, "weights")
    os.makedirs(wdir, exist_ok=True)
    manifest = {"format_version": 1, "model_config": config.to_json(),
                "quantization": quantization or {"method": "affine", "n_bits": 4, "seed": 0, "min_elements": 0},
                "tensors": {}}
    for name, t in tensors.items():
        s = sanitize_tensor_name(name)
        if not t.quantized:
            f = f"weights/{s}.bin"
            np.ascontiguousarray(t.data).tofile(os.path.join(path, f))
            manifest["tensors"][name] = {"format": "dense", "file": f, "shape": list(t.shape), "dtype": t.dtype}
            continue
        files = {"quantized_data_file": f"weights/{s}.qdata", "scales_file": f"weights/{s}.scale", "zeros_file": f"weights/{s}.zeros"}
        np.ascontiguousarray(t.data).tofile(os.path.join(path, files["quantized_data_file"]))
        np.ascontiguousarray(t.scale).tofile(os.path.join(path, files["scales_file"]))
        np.ascontiguousarray(t.zero_point).tofile(os.path.join(path, files["zeros_file"]))
        entry = {"format": "affine_dequantize", **files, "shape": list(t.shape), "bit_width": t.bit_width,
                 "group_size": t.group_size, "axis": t.axis if t.axis >= 0 else len(t.shape) - 1, "dtype": "uint8",
                 "scale_dtype": str(np.dtype(t.scale.dtype)), "zero_point_dtype": str(np.dtype(t.zero_point.dtype))}
        if t.awq_scales is not None:
            entry["awq_scales_file"] = f"weights/{s}.awq"
            np.ascontiguousarray(t.awq_scales).tofile(os.path.join(path, entry["awq_scales_file"]))
        manifest["tensors"][name] = entry
    with open(os.path.join(path, "manifest.json"), "w") as fh:
        json.dump(manifest, fh, indent=1)


QUANTIZED_SUFFIXES = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                      "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")


def quantize_to_gpu_bundle(path: str, provider, bit_width: int = 4, group_size: int = 128, awq_scales: dict | None = None,
                           min_elements: int = 0, device: int = 0) -> dict:
    """The compile step of the reference (affine quantization pass + bundle writer,
    crates/mil-rs/src/ir/passes/affine_quantize.rs:256-508, crates/ironmill-compile/src/weights/quantized.rs:852-1010,
    crates/ironmill-compile/src/gpu/bundle.rs:52-356) with the quantizer running on the GPU: every linear projection of the
    fp16 model behind `provider` is quantized and packed by the library's kernel (bit-exact with the reference's CPU
    quantizer: same groups, f32 scale and zero point, low-nibble-first packing), everything else is written dense, and
    the result is an ordinary `.ironml-gpu` directory.  awq_scales: optional {tensor name: fp16 [K]} per-input-channel
    scales, applied as W * s before quantization and stored beside the tensor.  Returns the manifest.

    No tile sidecar is written: the load-time repack into the kernels' tile stream is one pass of a GPU kernel over
    weights that are already on the device, far cheaper than reading a second copy of them from disk."""
    import torch

    from . import ops
    cfg: ModelConfig = provider.config()
    out = {}
    for name in provider.tensor_names():
        t = provider.tensor(name)
        quantize = (not t.quantized and name.endswith(QUANTIZED_SUFFIXES) and len(t.shape) == 2
                    and int(np.prod(t.shape)) >= min_elements)
        if not quantize:
            out[name] = t
            continue
        N, K = t.shape
        w = torch.from_numpy(np.ascontiguousarray(t.data, dtype=np.float16).reshape(N, K)).cuda(device)
        awq = None if not awq_scales or name not in awq_scales else np.ascontiguousarray(awq_scales[name], dtype=np.float16)
        packed, sc, zp = ops.quantize_affine(w, group_size, bit_width, None if awq is None else torch.from_numpy(awq).cuda(device))
        out[name] = WeightTensor(packed.cpu().numpy(), (N, K), "uint8", sc.cpu().numpy(), zp.cpu().numpy(), bit_width, group_size, 1, awq)
    write_gpu_bundle(path, cfg, out, {"method": "awq" if awq_scales else "affine", "n_bits": bit_width, "seed": 0, "min_elements": min_elements})
    return json.load(open(os.path.join(path, "manifest.json")))


class CudaBundleProvider:
    """WeightProvider over an `.ironml-gpu` directory: reads `manifest.json` up front and tensor files
    on demand (MetalBundleProvider, crates/ironmill-inference/src/metal/bundle.rs:22-92)."""

    def __init__(self, path: str):
        mpath = os.path.join(path, "manifest.json")
        if not os.path.isdir(path) or not os.path.exists(mpath):
            raise GpuBundleError(f"not a GPU bundle (no manifest.json): {path}")
        try:
            self.manifest = json.load(open(mpath))
        except json.JSONDecodeError as e:
            raise GpuBundleError(f"manifest.json: {e}") from e
        if self.manifest.get("format_version") != 1:
            raise GpuBundleError(f"unsupported format_version {self.manifest.get('format_version')}")
        self.path = path
        self._config = ModelConfig.from_json(self.manifest.get("model_config"))
        self._tensors = self.manifest.get("tensors") or {}

    def config(self) -> ModelConfig:
        return self._config

    def tensor_names(self):
        return list(self._tensors)

    def has_tensor(self, name: str) -> bool:
        return name in self._tensors

    def _read(self, rel: str, dtype, count: int | None = None) -> np.ndarray:
        p = os.path.join(self.path, rel)
        if not os.path.exists(p):
            raise GpuBundleError(f"missing weight file {rel}")
        a = np.fromfile(p, dtype=dtype)
        if count is not None and a.size != count:
            raise GpuBundleError(f"{rel}: expected {count} elements of {np.dtype(dtype)}, found {a.size}")
        return a

    def tensor(self, name: str) -> WeightTensor:
        e = self._tensors.get(name)
        if e is None:
            raise GpuBundleError(f"tensor not found: {name}")
        fmt = e.get("format")
        shape = tuple(e["shape"])
        n = int(np.prod(shape))
        if fmt == "dense":
            dt = _DTYPES.get(e["dtype"])
            if dt is None:
                raise GpuBundleError(f"{name}: unsupported dtype {e['dtype']}")
            return WeightTensor(self._read(e["file"], dt, n).reshape(shape), shape, e["dtype"])
        if fmt == "affine_dequantize":
            bits, gs = int(e["bit_width"]), int(e["group_size"])
            if bits not in (4, 8):
                raise GpuBundleError(f"{name}: bit_width {bits} is not supported")
            if e.get("g_idx_file"):
                raise GpuBundleError(f"{name}: GPTQ g_idx reordering is not supported by this backend")
            K = shape[-1]
            rows = n // K
            G = -(-K // gs)
            # crates/ironmill-core/src/gpu/bundle.rs:376-399: absent dtype fields default to float16
            sdt = _DTYPES[e.get("scale_dtype") or "float16"]
            zdt = _DTYPES[e.get("zero_point_dtype") or "float16"]
            codes = self._read(e["quantized_data_file"], np.uint8, (n + 1) // 2 if bits == 4 else n)
            scale = self._read(e["scales_file"], sdt, rows * G).reshape(rows, G)
            zp = self._read(e["zeros_file"], zdt, rows * G).reshape(rows, G)
            awq = self._read(e["awq_scales_file"], np.float16, K) if e.get("awq_scales_file") else None
            return WeightTensor(codes, shape, "uint8", scale, zp, bits, gs, int(e.get("axis", len(shape) - 1)), awq)
        raise GpuBundleError(f"{name}: tensor format '{fmt}' is not supported by this backend")
