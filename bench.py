#!/usr/bin/env python
"""Benchmark of the quantized decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Workloads (synthetic, seeded; shapes of the Llama-3-8B-shaped
decode config):

  matvec  one step = one pass over the four INT4 g128 projection launches of a decoder layer at
          batch 1 with AWQ scales: fused QKV 4096->6144, o 4096->4096, fused gate+up+SiLU
          4096->2x14336, down 14336->4096.  Metric: algorithmic HBM GB/s (packed codes + fp16
          scale/zero + activations in/out, the byte count the reference's own kernel bandwidth
          benchmark uses).  Each step reads a different copy of the weights out of a rotation
          larger than L2.

`--impl reference` times the CPU restatement of the reference's own CPU path (the oracle) on the
host cores for the same workload, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama-3-8B-shaped projections: (name, N, K, kind)
L8_SHAPES = [("qkv", 6144, 4096, "plain"), ("o", 4096, 4096, "plain"),
             ("gate_up", 14336, 4096, "ffn"), ("down", 4096, 14336, "plain")]
GS = 128


def matvec_bytes(N, K, B=1, awq=True, bits=4):
    """Algorithmic bytes of one affine matvec (crates/ironmill-bench/examples/kernel_bandwidth_bench.rs:350-358):
    packed codes + fp16 scale and zero per group + fp16 input + fp16 output (+ fp16 AWQ vector)."""
    return N * K * bits // 8 + 2 * (N * K // GS) * 2 + B * K * 2 + B * N * 2 + (K * 2 if awq else 0)


def shape_bytes(name, N, K, kind):
    if kind == "ffn":   # two [N,K] matrices share x; output is N halves
        return 2 * (N * K // 2 + 2 * (N * K // GS) * 2) + K * 2 + N * 2 + K * 2
    return matvec_bytes(N, K)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ----------------------------------------------------------------------------- synthetic weights on the GPU
def gpu_layer_copy(dev, seed):
    """One copy of the four projections, quantized ON the GPU with the library's own quantizer."""
    import torch

    from ironmill_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = {}
    for name, N, K, kind in L8_SHAPES:
        awq = torch.rand(K, generator=g, device="cuda") * 1.5 + 0.5
        awq = awq.half()
        mats = []
        for _ in range(2 if kind == "ffn" else 1):
            w = (torch.randn((N, K), generator=g, device="cuda") * 0.02).half()
            packed, s, z = ops.quantize_affine(w, GS, 4, awq)
            mats.append(ops.AffineWeight(dev, packed, s, z, N, K, GS, 4, awq=awq))
            del w, packed, s, z
        out[name] = mats
    return out


def run_ours(args, rank, world):
    import torch
    import torch.distributed as dist

    from ironmill_b200 import ops

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = ops.Device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    ncopies = 4   # 4 x 116 MB of weights > 126 MB of L2: no step finds its weights cached
    copies = [gpu_layer_copy(dev, 100 + rank * 10 + i) for i in range(ncopies)]
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    xs = {K: torch.randn((1, K), generator=g, device="cuda").half() for K in (4096, 14336)}
    ys = {name: torch.empty((1, N), dtype=torch.float16, device="cuda") for name, N, K, kind in L8_SHAPES}
    step_bytes = sum(shape_bytes(*s) for s in L8_SHAPES)
    launches_per_step = len(L8_SHAPES)

    def step(i, ev=None):
        cp = copies[i % ncopies]
        for name, N, K, kind in L8_SHAPES:
            if ev is not None and name == "gate_up":
                ev[0].record()
            if kind == "ffn":
                ops.ffn_gate_up_act(cp[name][0], cp[name][1], xs[K], out=ys[name])
            else:
                ops.matvec_affine(cp[name][0], xs[K], out=ys[name])
            if ev is not None and name == "gate_up":
                ev[1].record()

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    for i in range(args.steps):
        step(i, evs[i])
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    dom_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the host-buffer call: x from host memory in, y back to host, per projection
    e2e_steps = max(3, min(args.steps, 50))
    xh = {K: np.random.default_rng(1).standard_normal((1, K)).astype(np.float16) for K in (4096, 14336)}
    plain = [s for s in L8_SHAPES if s[3] == "plain"]
    e2e_bytes = sum(shape_bytes(*s) for s in plain)
    for i in range(2):
        for name, N, K, kind in plain:
            ops.matvec_affine_host(copies[i % ncopies][name][0], xh[K])
    torch.cuda.synchronize()
    w0 = time.perf_counter()
    for i in range(e2e_steps):
        for name, N, K, kind in plain:
            ops.matvec_affine_host(copies[i % ncopies][name][0], xh[K])
    e2e_s = time.perf_counter() - w0
    h2d = sum(K * 2 for _, N, K, _ in plain)
    d2h = sum(N * 2 for _, N, K, _ in plain)

    if rank != 0:
        return
    peak, peak_src = measured_peaks()
    gate_up = [s for s in L8_SHAPES if s[0] == "gate_up"][0]
    dom_bytes = shape_bytes(*gate_up)
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    out = {
        "metric": "matvec HBM GB/s (INT4 g128 affine, Llama-3-8B projection shapes, batch 1)",
        "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u4 codes x i16 activations, f32 fix-up", "data": "synthetic",
        "config": {"workload": "int4_g128_matvec_sweep_llama3_8b_shapes_b1_awq",
                   "shapes": [[n, N, K] for n, N, K, _ in L8_SHAPES], "group_size": GS,
                   "l2_policy": f"rotation over {ncopies} weight copies ({ncopies * step_bytes >> 20} MiB) larger than L2",
                   "parallelism": f"replicas x{world}" if world > 1 else "single"},
        "roofline": {"bound": "hbm", "kernel": "matvec_kernel<4,gate_up_act> 4096->2x14336", "achieved": round(achieved, 1),
                     "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_source": peak_src,
                     "bytes_per_launch": dom_bytes, "us_per_launch": round(dom_ms * 1e3, 3), "traffic": None},
        "e2e": {"value": round(world * e2e_bytes * e2e_steps / e2e_s / 1e9, 3), "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "host-buffer matvec calls (qkv, o, down): copy x in, launch, copy y out, synchronise"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if world == 1:
        out["cpu_baseline"] = cpu_baseline(sample_only=True)
    print(json.dumps(out))


# ----------------------------------------------------------------------------- CPU arm
def cpu_baseline(sample_only: bool):
    """The CPU restatement of the reference's quantize + dequantised matvec (the oracle), timed on
    the host cores on a bounded sample: W [4096,4096] -> INT4 g128 + y = dequant(W) x, batch 1."""
    from oracle import oracle as orc
    threads = orc.max_threads()
    rng = np.random.default_rng(0)
    N = K = 4096
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    x = rng.standard_normal((1, K)).astype(np.float16)
    t0 = time.perf_counter()
    codes, scales, zps = orc.quantize_groups(w, GS, 4, threads=threads)
    packed = orc.pack_int4(codes)
    tq = time.perf_counter() - t0
    s16, z16 = orc.f32_to_f16(scales), orc.f32_to_f16(zps)
    reps = 0
    t0 = time.perf_counter()
    while True:
        orc.matvec_affine(packed, s16, z16, x, N, K, GS, 4, threads=threads)
        reps += 1
        if time.perf_counter() - t0 > (3.0 if sample_only else 8.0):
            break
    tm = (time.perf_counter() - t0) / reps
    gbs = matvec_bytes(N, K, awq=False) / tm / 1e9
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"o_proj-sized 4096x4096 INT4 g128 matvec, batch 1, {reps} repetitions, OpenMP {threads} threads; "
                      f"quantize+pack of the same matrix took {tq * 1e3:.0f} ms",
            "quantize_ms": round(tq * 1e3, 1), "matvec_ms": round(tm * 1e3, 3)}


def run_reference(args, rank, world):
    if rank != 0:
        return
    t0 = time.perf_counter()
    res = []
    for _ in range(max(1, min(args.steps, 3))):
        res.append(cpu_baseline(sample_only=False))
    cb = res[-1]
    v = float(np.mean([r["value"] for r in res]))
    out = {"impl": "reference", "metric": "matvec HBM GB/s (INT4 g128 affine, Llama-3-8B projection shapes, batch 1)",
           "value": round(v, 3), "unit": "GB/s", "n_gpus": world, "steps": len(res), "warmup": 0,
           "ms_per_step": round((time.perf_counter() - t0) / len(res) * 1e3, 2), "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": "int4_g128_matvec_sweep_llama3_8b_shapes_b1_awq", "group_size": GS},
           "cpu_baseline": dict(cb, value=round(v, 3)),
           "e2e": {"value": round(v, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world)


if __name__ == "__main__":
    main()
