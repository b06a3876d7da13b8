"""CPU checks of the oracle model itself (test infrastructure): its deviation switches do what they say on a tiny
model, and the default run is deterministic."""
import numpy as np

from ironmill_b200.bundle import ModelConfig
from oracle import oracle as orc
from tests.oracle_model import OracleModel, synth_model


def _tiny():
    cfg = ModelConfig(architecture="qwen3", hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, vocab_size=300, max_position_embeddings=64, rms_norm_eps=1e-6,
                      rope_theta=1e6, tie_word_embeddings=False)
    return cfg, synth_model(cfg, seed=9, awq=True, gamma_jitter=0.1, threads=2), orc.TqConstants(128, 8, seed=42)


def _run(cfg, tensors, tqc, **kw):
    m = OracleModel(cfg, tensors, tqc, 32, **kw)
    out = [m.forward(np.arange(7, dtype=np.uint32))]
    for t in (5, 17, 250):
        out.append(m.forward([t]))
    return np.stack(out)


def test_reference_run_is_deterministic_and_switches_move_it_a_little():
    cfg, tensors, tqc = _tiny()
    base = _run(cfg, tensors, tqc)
    assert np.array_equal(base, _run(cfg, tensors, tqc))
    for dev in ("kv_unrounded", "ffn_unrounded", "act_q16", "act_q24", "sum_order", "prefill_matvec"):
        d = _run(cfg, tensors, tqc, deviations=(dev,))
        diff = np.abs(d - base).max()
        assert 0.0 < diff < 5e-2, (dev, diff)      # a rounding-level change, and a real one
        if dev in ("kv_unrounded", "ffn_unrounded", "act_q16", "act_q24"):
            assert np.array_equal(d[0], base[0]), dev   # decode-only switches leave the prefill alone


def test_layer_zero_and_int8_take_no_fused_projection():
    # with 8-bit weights the reference has no fused kernels: the decode-time switches must change nothing
    cfg, _, tqc = _tiny()
    tensors = synth_model(cfg, seed=9, bits=8, threads=2)
    base = _run(cfg, tensors, tqc)
    for dev in ("kv_unrounded", "ffn_unrounded"):
        assert np.array_equal(base, _run(cfg, tensors, tqc, deviations=(dev,)))


def test_fp16_kv_attention_restatement_against_plain_softmax_and_its_split_form():
    # fused_sdpa (tiles of 32, conditional rescale) and fused_sdpa_split + reduce (tiles of 8) against a float64 softmax
    rng = np.random.default_rng(4)
    nh, nkv, hd, ms, T, base = 4, 2, 128, 300, 3, 257
    q = rng.standard_normal((T, nh, hd)).astype(np.float16)
    K = rng.standard_normal((nkv, ms, hd)).astype(np.float16)
    V = rng.standard_normal((nkv, ms, hd)).astype(np.float16)
    sc = 1.0 / np.sqrt(hd)
    one = orc.sdpa_f16(q, K, V, sc, nh, nkv, hd, ms, base, 0).astype(np.float64)
    split = orc.sdpa_f16(q, K, V, sc, nh, nkv, hd, ms, base, 5).astype(np.float64)
    ref = np.zeros_like(one)
    for t in range(T):
        for h in range(nh):
            n = base + t + 1
            s = (K[h // 2, :n].astype(np.float64) @ q[t, h].astype(np.float64)) * sc
            w = np.exp(s - s.max())
            ref[t, h] = (w / w.sum()) @ V[h // 2, :n].astype(np.float64)
    assert np.abs(one - ref).max() <= 1e-3 and np.abs(split - ref).max() <= 1e-3   # one fp16 rounding of values of order 0.1-1
    assert np.abs(one - split).max() <= 5e-4


def test_model_with_an_fp16_kv_cache_stays_close_to_the_turboquant_model():
    # TurboQuant off (kv_f16): same schedule, attention over unquantized rows; the 8-bit cache costs a few 1e-2 of logit
    cfg, tensors, tqc = _tiny()
    a = _run(cfg, tensors, tqc)
    b = _run(cfg, tensors, None, kv_f16=True)
    assert np.array_equal(b, _run(cfg, tensors, None, kv_f16=True))
    assert 0.0 < np.abs(a - b).max() < 0.25
