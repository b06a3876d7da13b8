"""Tensor-parallel engine on 2, 4 or 8 GPUs: logits of the sharded model against the CPU oracle model and against the
single-GPU engine.  Runs on the largest power of two of visible GPUs (IM_TEST_TP_WORLD overrides); skipped with one GPU."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ironmill_b200.bundle import ModelConfig
        from ironmill_b200.engine import CudaConfig, CudaInference
        from oracle import oracle as orc
        from tests.oracle_model import DictProvider, OracleModel, synth_model
        nkv = max(2, world)   # KV heads are split across the ranks
        cfg = ModelConfig(architecture="llama", hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4 * nkv,
                          num_key_value_heads=nkv, head_dim=128, vocab_size=1000, rms_norm_eps=1e-5, rope_theta=5e5)
        tensors = synth_model(cfg, seed=9, awq=True)
        tqc = orc.TqConstants(128, 8, seed=42)
        eng = CudaInference(CudaConfig(max_seq_len=320, tp_world=world, tp_rank=rank, device=rank))
        eng.load_weights(DictProvider(cfg, tensors), tq_signs=tqc.signs, tq_qjl=tqc.qjl)
        ids = [CudaInference.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        eng.tp_init(ids[0])
        prompt = np.arange(7, dtype=np.uint32) * 13 % 1000
        outs = [eng.prefill(prompt)]
        steps = (5, 17, 400, 3, 999, 12, 77, 250)   # batch-1 steps: the whole-token kernel with its cross-rank barriers when enabled
        for t in steps:
            outs.append(eng.decode_step(t))
        eng.reset()
        long_prompt = (np.arange(280, dtype=np.uint32) * 29 + 3) % 1000   # a full 256-token chunk and a remainder on the tensor-core GEMM
        outs.append(eng.prefill(long_prompt))
        for t in steps[:3]:   # decode on top of the long prefill: attention past 256 positions
            outs.append(eng.decode_step(t))
        if rank == 0:
            single = CudaInference(CudaConfig(max_seq_len=320, device=0))
            single.load_weights(DictProvider(cfg, tensors), tq_signs=tqc.signs, tq_qjl=tqc.qjl)
            oracle = OracleModel(cfg, tensors, tqc, 320)
            refs = [single.prefill(prompt)] + [single.decode_step(t) for t in steps]
            orefs = [oracle.forward(prompt)] + [oracle.forward([t]) for t in steps]
            single.reset()
            oracle = OracleModel(cfg, tensors, tqc, 320)
            refs += [single.prefill(long_prompt)] + [single.decode_step(t) for t in steps[:3]]
            orefs += [oracle.forward(long_prompt)] + [oracle.forward([t]) for t in steps[:3]]
            err = max(float(np.abs(a - b).max()) for a, b in zip(outs, refs))
            ret[0] = err
            ret['oracle_err'] = max(float(np.abs(a - b).max()) for a, b in zip(outs, orefs))
            ret['peer'] = eng.tp_peer_allreduce()
            ret['token_kernel'] = eng.token_kernel()
        dist.barrier()
    except Exception as e:  # noqa: BLE001
        ret[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def test_tp_matches_single_gpu():
    have = torch.cuda.device_count()
    world = int(os.environ.get("IM_TEST_TP_WORLD", "0")) or (8 if have >= 8 else 4 if have >= 4 else 2)
    if have < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert isinstance(ret.get(0), float) and ret[0] <= 5e-2, dict(ret)
    assert ret.get('oracle_err', 1.0) <= 5e-2, dict(ret)          # against the CPU oracle model, the stated decode gate
    print('one-shot peer all-reduce in use:', ret.get('peer'), '| whole-token kernel across ranks:', ret.get('token_kernel'))
    assert all(r not in ret for r in range(1, world)), dict(ret)
