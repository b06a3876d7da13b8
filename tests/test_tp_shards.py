"""Tensor-parallel shard arithmetic on CPU (no GPU): two gloo ranks cut their shards with the library's own host
helpers, compute their part of one decoder layer's projections with the CPU oracle, and exchange exactly the
collectives the GPU engine issues (one all-reduce after each row-split projection); the result must equal the
unsharded oracle."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _shard(lib, cfg_struct, suffix, qw):
    """qw: tests.helpers.QWeight (full tensor) -> dict with this rank's shard."""
    from ironmill_b200._lib import check, vp
    r0, nr, c0, nc = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    check(lib.im_cuda_tp_shard_rect(C.byref(cfg_struct), suffix.encode(), C.byref(r0), C.byref(nr), C.byref(c0), C.byref(nc)))
    nr_, nc_ = nr.value, nc.value
    G = nc_ // 128
    q = np.zeros(nr_ * nc_ // 2, np.uint8)
    s = np.zeros((nr_, G), np.float32)
    z = np.zeros((nr_, G), np.float32)
    awq = np.zeros(nc_, np.float16)
    check(lib.im_cuda_tp_shard_affine(vp(qw.packed), vp(qw.scales), vp(qw.zps), 1, vp(qw.awq), qw.N, qw.K, 128, 4, r0.value, nr_,
                                      c0.value, nc_, vp(q), vp(s), vp(z), vp(awq)))
    return dict(q=q, s=s, z=z, awq=awq, N=nr_, K=nc_, r0=r0.value, c0=c0.value)


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ironmill_b200 import build
        from ironmill_b200.engine import _CModelConfig
        from oracle import oracle as orc
        from tests import helpers as H
        lib = C.CDLL(build.LIB)
        lib.im_cuda_last_error.restype = C.c_char_p
        Hd, I, nh, nkv, hd = 512, 1024, 4, 2, 128
        cfg = _CModelConfig(1, Hd, I, nh, nkv, hd, 100, 64, 1, 1e-5, 0.0, 0.0, 1e4, 0, 0, 0, 8, 42, world, rank)
        ws = {"self_attn.q_proj.weight": H.QWeight(nh * hd, Hd, awq=True, seed=1, name="q"),
              "self_attn.o_proj.weight": H.QWeight(Hd, nh * hd, awq=True, seed=1, name="o"),
              "mlp.gate_proj.weight": H.QWeight(I, Hd, awq=True, seed=1, name="g"),
              "mlp.down_proj.weight": H.QWeight(Hd, I, awq=True, seed=1, name="d")}
        ws["mlp.up_proj.weight"] = H.QWeight(I, Hd, seed=1, name="u", awq_vec=ws["mlp.gate_proj.weight"].awq)
        sh = {k: _shard(lib, cfg, k, v) for k, v in ws.items()}
        f16 = orc.f32_to_f16

        def mv(w, x):      # full or sharded matvec through the oracle
            if isinstance(w, dict):
                return orc.matvec_affine(w["q"], f16(w["s"]), f16(w["z"]), x, w["N"], w["K"], 128, 4, awq=w["awq"])
            return orc.matvec_affine(w.packed, w.scales_f16, w.zps_f16, x, w.N, w.K, 128, 4, awq=w.awq)

        x = H.make_x(1, Hd, seed=3)
        # column-parallel q: each rank owns nh/world heads; row-parallel o consumes exactly those columns
        q_full = mv(ws["self_attn.q_proj.weight"], x)
        q_loc = mv(sh["self_attn.q_proj.weight"], x)
        r0 = sh["self_attn.q_proj.weight"]["r0"]
        assert (q_loc.view(np.uint16) == q_full[:, r0:r0 + q_loc.shape[1]].view(np.uint16)).all()
        assert sh["self_attn.o_proj.weight"]["c0"] == r0, "o_proj columns must line up with this rank's q heads"
        o_part = mv(sh["self_attn.o_proj.weight"], q_loc).astype(np.float32)
        t = torch.from_numpy(o_part)
        dist.all_reduce(t)                      # the engine: ncclAllReduce(fp16 sum) after o_proj
        o_full = mv(ws["self_attn.o_proj.weight"], q_full).astype(np.float32)
        assert np.abs(t.numpy() - o_full).max() <= 2e-3 * np.abs(o_full).max() + 1e-3
        # FFN: gate/up column-parallel, down row-parallel
        g, u = sh["mlp.gate_proj.weight"], sh["mlp.up_proj.weight"]
        act = orc.ffn_gate_up_act(g["q"], f16(g["s"]), f16(g["z"]), u["q"], f16(u["s"]), f16(u["z"]), x, g["N"], Hd, 128, 4, awq=g["awq"])
        gw, uw = ws["mlp.gate_proj.weight"], ws["mlp.up_proj.weight"]
        act_full = orc.ffn_gate_up_act(gw.packed, gw.scales_f16, gw.zps_f16, uw.packed, uw.scales_f16, uw.zps_f16, x, I, Hd, 128, 4, awq=gw.awq)
        assert (act.view(np.uint16) == act_full[:, g["r0"]:g["r0"] + g["N"]].view(np.uint16)).all()
        assert sh["mlp.down_proj.weight"]["c0"] == g["r0"]
        d_part = torch.from_numpy(mv(sh["mlp.down_proj.weight"], act).astype(np.float32))
        dist.all_reduce(d_part)
        d_full = mv(ws["mlp.down_proj.weight"], act_full).astype(np.float32)
        assert np.abs(d_part.numpy() - d_full).max() <= 2e-3 * np.abs(d_full).max() + 1e-3
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        ret[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def test_two_rank_shards_reproduce_the_unsharded_layer():
    from ironmill_b200 import build
    build.build()
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}, dict(ret)


def test_shard_rect_rejects_misaligned_columns():
    from ironmill_b200 import build
    lib = C.CDLL(build.build())
    lib.im_cuda_last_error.restype = C.c_char_p
    q = np.zeros(4 * 256 // 2, np.uint8)
    s = np.zeros((4, 2), np.float32)
    out = np.zeros(4 * 64, np.uint8)
    rc = lib.im_cuda_tp_shard_affine(q.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p), 1, None,
                                     4, 256, 128, 4, 0, 4, 64, 128, out.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p),
                                     s.ctypes.data_as(C.c_void_p), None)
    assert rc == -1 and b"aligned" in lib.im_cuda_last_error()
