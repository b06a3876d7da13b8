"""fp16 (unquantized) KV cache: kv_scatter + attention against the CPU oracle's restatement of the reference's
fused_sdpa / prefill_attention_v2 / fused_sdpa_split + fused_sdpa_reduce, and a whole model decoding with TurboQuant off."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

# tolerance: the same fp16 inputs, f32 scores and sums in another order, one fp16 rounding of the output
TOL = 2e-3


@pytest.fixture(scope="module")
def dev():
    from ironmill_b200 import ops
    return ops.Device(0)


def _caches(nkv, max_seq, seed):
    rng = H.rng_for("kv16", seed)
    k = (rng.standard_normal((nkv, max_seq, 128)) * 0.7).astype(np.float16)
    v = rng.standard_normal((nkv, max_seq, 128)).astype(np.float16)
    return k, v


@pytest.mark.parametrize("nh,nkv", [(4, 4), (4, 2), (8, 2), (8, 1)])
@pytest.mark.parametrize("ctx,splits", [(1, 0), (31, 1), (33, 0), (255, 0), (256, 0), (257, 3), (1000, 0), (1000, 7), (3000, 0)])
def test_decode_attention_matches_the_oracle(dev, nh, nkv, ctx, splits):
    from ironmill_b200 import ops
    max_seq = 3072
    k, v = _caches(nkv, max_seq, ctx + nh)
    q = H.rng_for("kv16-q", ctx).standard_normal((1, nh, 128)).astype(np.float16)
    scale = 1.0 / np.sqrt(128.0)
    out = ops.sdpa_f16(dev, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), scale, nh, nkv, max_seq,
                       ctx - 1, num_splits=splits).cpu().numpy()
    # the reference takes the split pair from 256 positions on; both forms agree far inside the tolerance
    ref = orc.sdpa_f16(q, k, v, scale, nh, nkv, 128, max_seq, ctx - 1, num_splits=0 if ctx < 256 else max(2, -(-ctx // 256)))
    assert H.rel_err(out, ref) <= TOL, (nh, nkv, ctx, splits)


def test_prefill_is_causal_and_batched_sequences_use_their_own_positions(dev):
    from ironmill_b200 import ops
    nh, nkv, max_seq, T = 8, 2, 512, 37
    scale = 0.09
    # one sequence, 37 new tokens after 100 cached ones
    k, v = _caches(nkv, max_seq, 5)
    q = H.rng_for("kv16-qp").standard_normal((T, nh, 128)).astype(np.float16)
    out = ops.sdpa_f16(dev, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), scale, nh, nkv, max_seq, 100).cpu().numpy()
    ref = orc.sdpa_f16(q, k, v, scale, nh, nkv, 128, max_seq, 100)
    assert H.rel_err(out, ref) <= TOL
    # three sequences at different positions, one token each
    pos = np.array([5, 300, 77], dtype=np.int32)
    ks, vs = zip(*[_caches(nkv, max_seq, 20 + i) for i in range(3)])
    qb = H.rng_for("kv16-qb").standard_normal((3, nh, 128)).astype(np.float16)
    outb = ops.sdpa_f16(dev, torch.from_numpy(qb).cuda(), torch.from_numpy(np.stack(ks)).cuda(), torch.from_numpy(np.stack(vs)).cuda(), scale, nh, nkv,
                        max_seq, 0, nseq=3, pos_dev=torch.from_numpy(pos).cuda()).cpu().numpy()
    for i in range(3):
        refi = orc.sdpa_f16(qb[i:i + 1], ks[i], vs[i], scale, nh, nkv, 128, max_seq, int(pos[i]))
        assert H.rel_err(outb[i:i + 1], refi) <= TOL, i


@pytest.mark.parametrize("nh,nkv", [(4, 4), (4, 2), (8, 2), (8, 1)])
@pytest.mark.parametrize("base,T", [(0, 16), (0, 130), (77, 50), (500, 300)])
def test_prefill_tensor_core_pass_matches_the_oracle(dev, nh, nkv, base, T):
    # chunks of 16 tokens and more of one sequence: the causal tensor-core pass (sdpa16_prefill_kernel); 1, 2, 4 and 8
    # query heads per KV head; cached prefixes of 0, 77 and 500 positions
    from ironmill_b200 import ops
    max_seq = base + T + 7
    k, v = _caches(nkv, max_seq, base + T + nh)
    q = H.rng_for("kv16-qpf", T).standard_normal((T, nh, 128)).astype(np.float16)
    out = ops.sdpa_f16(dev, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), 0.0884, nh, nkv, max_seq, base).cpu().numpy()
    ref = orc.sdpa_f16(q, k, v, 0.0884, nh, nkv, 128, max_seq, base)
    assert H.rel_err(out, ref) <= TOL, (nh, nkv, base, T)


def test_kv_scatter_writes_the_rows_of_the_new_tokens(dev):
    from ironmill_b200 import ops
    nkv, max_seq, T = 2, 64, 5
    proj = H.rng_for("kv16-s").standard_normal((2 * T, nkv, 128)).astype(np.float16)
    cache = torch.zeros((2, nkv, max_seq, 128), dtype=torch.float16, device="cuda")
    pos = torch.tensor([3, 40], dtype=torch.int32, device="cuda")
    ops.kv_scatter_f16(torch.from_numpy(proj).cuda(), cache, 2, T, nkv, max_seq, 0, pos_dev=pos)
    got = cache.cpu().numpy()
    want = np.zeros_like(got)
    for s, p0 in enumerate((3, 40)):
        for t in range(T):
            want[s, :, p0 + t] = proj[s * T + t]
    assert np.array_equal(got, want)   # a copy: bit-exact


def test_long_context(dev):
    from ironmill_b200 import ops
    nh, nkv, max_seq, ctx = 4, 1, 32768, 32768
    k, v = _caches(nkv, max_seq, 99)
    q = H.rng_for("kv16-ql").standard_normal((1, nh, 128)).astype(np.float16)
    scale = 1.0 / np.sqrt(128.0)
    out = ops.sdpa_f16(dev, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), scale, nh, nkv, max_seq, ctx - 1).cpu().numpy()
    ref = orc.sdpa_f16(q, k, v, scale, nh, nkv, 128, max_seq, ctx - 1, num_splits=128)
    assert H.rel_err(out, ref) <= TOL


@pytest.mark.parametrize("arch", ["llama", "qwen3"])
def test_model_with_turboquant_off_matches_the_oracle(arch):
    """MetalConfig.enable_turboquant = false: prefill (GEMM form, causal attention over fp16 rows), then decode steps
    (per-kernel schedule), then a second sequence through the batching interface."""
    from ironmill_b200.bundle import ModelConfig
    from ironmill_b200.engine import CudaConfig, CudaInference
    from tests.oracle_model import DictProvider, OracleModel, synth_model
    cfg = ModelConfig(architecture=arch, hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=128, vocab_size=400, max_position_embeddings=512, rms_norm_eps=1e-6,
                      rope_theta=1e6, tie_word_embeddings=False)
    tensors = synth_model(cfg, seed=31, awq=(arch == "llama"))
    eng = CudaInference(CudaConfig(max_seq_len=384, max_batch=2).without_turboquant())
    eng.load_weights(DictProvider(cfg, tensors))
    ref = OracleModel(cfg, tensors, None, 384, kv_f16=True)
    prompt = H.rng_for("kv16-m").integers(0, 400, 270).astype(np.uint32)   # the decode steps cross into the split form
    a, b = eng.prefill(prompt), ref.forward(prompt)
    assert np.abs(a - b).max() <= 5e-2
    agree = 0
    for i in range(12):
        tok = int(orc.argmax(b))
        a, b = eng.decode_step(tok), ref.forward(np.array([tok], dtype=np.uint32))
        assert np.abs(a - b).max() <= 5e-2, i
        agree += int(np.argmax(a) == orc.argmax(b))
    assert agree >= 11
    # a second sequence beside the first (cache slots with their own positions)
    eng.reset()
    s0 = eng.add_sequence(prompt[:40])
    s1 = eng.add_sequence(prompt[100:117])
    r0, r1 = OracleModel(cfg, tensors, None, 384, kv_f16=True), OracleModel(cfg, tensors, None, 384, kv_f16=True)
    l0, l1 = r0.forward(prompt[:40]), r1.forward(prompt[100:117])
    out = dict(eng.batch_decode_step())
    assert sorted(out) == sorted([s0, s1])
    w0, w1 = r0.forward(np.array([orc.argmax(l0)], dtype=np.uint32)), r1.forward(np.array([orc.argmax(l1)], dtype=np.uint32))
    assert np.abs(out[s0] - w0).max() <= 5e-2 and np.abs(out[s1] - w1).max() <= 5e-2
