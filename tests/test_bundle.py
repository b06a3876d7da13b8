"""`.ironml-gpu` bundle reader/writer (host logic, no GPU): round trip and the error behaviour of
the reference's bundle provider tests (crates/ironmill-inference/src/metal/bundle.rs:101-233)."""
import json
import os

import numpy as np
import pytest

from ironmill_b200.bundle import CudaBundleProvider, GpuBundleError, ModelConfig, WeightTensor, sanitize_tensor_name, write_gpu_bundle
from oracle import oracle as orc


def _cfg():
    return ModelConfig(architecture="qwen3", hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=128, vocab_size=100,
                       max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=1e6)


def _tensors():
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((8, 256)) * 0.02).astype(np.float16)
    awq = rng.uniform(0.5, 2, 256).astype(np.float16)
    codes, s, z = orc.quantize_groups(w, 128, 4, awq=awq)
    return {"model.norm.weight": WeightTensor(np.ones(256, np.float16), (256,), "float16"),
            "model.layers.0.mlp.up_proj.weight": WeightTensor(orc.pack_int4(codes), (8, 256), "uint8", s, z, 4, 128, 1, awq),
            "model.layers.0.mlp.gate_proj.weight": WeightTensor(codes.reshape(-1), (8, 256), "uint8", orc.f32_to_f16(s), orc.f32_to_f16(z), 8, 128, 1, None)}


def test_round_trip(tmp_path):
    p = str(tmp_path / "m.ironml-gpu")
    t = _tensors()
    write_gpu_bundle(p, _cfg(), t)
    assert os.path.exists(os.path.join(p, "weights", "model_layers_0_mlp_up_proj_weight.qdata"))
    prov = CudaBundleProvider(p)
    c = prov.config()
    assert c.architecture == "qwen3" and c.hidden_size == 256 and c.has_qk_norm and abs(c.attn_scale - 128 ** -0.5) < 1e-7
    assert sorted(prov.tensor_names()) == sorted(t)
    for name, src in t.items():
        got = prov.tensor(name)
        assert got.shape == src.shape and (got.data.reshape(-1) == np.asarray(src.data).reshape(-1)).all()
        if src.quantized:
            assert got.bit_width == src.bit_width and got.group_size == 128
            assert got.scale.dtype == src.scale.dtype and (got.scale == src.scale).all() and (got.zero_point == src.zero_point).all()
            assert (got.awq_scales is None) == (src.awq_scales is None)
    m = json.load(open(os.path.join(p, "manifest.json")))
    assert m["format_version"] == 1 and m["tensors"]["model.layers.0.mlp.up_proj.weight"]["scale_dtype"] == "float32"


def test_sanitize():
    assert sanitize_tensor_name("model.layers.0/x.weight") == "model_layers_0_x_weight"


def test_missing_dtype_fields_default_to_fp16(tmp_path):
    p = str(tmp_path / "m.ironml-gpu")
    write_gpu_bundle(p, _cfg(), _tensors())
    mp = os.path.join(p, "manifest.json")
    m = json.load(open(mp))
    e = m["tensors"]["model.layers.0.mlp.gate_proj.weight"]
    del e["scale_dtype"], e["zero_point_dtype"]
    json.dump(m, open(mp, "w"))
    assert CudaBundleProvider(p).tensor("model.layers.0.mlp.gate_proj.weight").scale.dtype == np.float16


def test_errors(tmp_path):
    with pytest.raises(GpuBundleError):
        CudaBundleProvider(str(tmp_path / "nope"))
    p = str(tmp_path / "m.ironml-gpu")
    write_gpu_bundle(p, _cfg(), _tensors())
    prov = CudaBundleProvider(p)
    assert not prov.has_tensor("missing")
    with pytest.raises(GpuBundleError):
        prov.tensor("missing")
    os.remove(os.path.join(p, "weights", "model_norm_weight.bin"))
    with pytest.raises(GpuBundleError):
        prov.tensor("model.norm.weight")
    # truncated file
    q = os.path.join(p, "weights", "model_layers_0_mlp_up_proj_weight.qdata")
    open(q, "wb").write(b"\0" * 10)
    with pytest.raises(GpuBundleError):
        prov.tensor("model.layers.0.mlp.up_proj.weight")
    # unsupported tensor format and manifest version
    mp = os.path.join(p, "manifest.json")
    m = json.load(open(mp))
    m["tensors"]["x"] = {"format": "lut_to_dense", "shape": [1]}
    json.dump(m, open(mp, "w"))
    with pytest.raises(GpuBundleError):
        CudaBundleProvider(p).tensor("x")
    m["format_version"] = 2
    json.dump(m, open(mp, "w"))
    with pytest.raises(GpuBundleError):
        CudaBundleProvider(p)
    m["format_version"] = 1
    del m["model_config"]["hidden_size"]
    json.dump(m, open(mp, "w"))
    with pytest.raises(GpuBundleError):
        CudaBundleProvider(p)
