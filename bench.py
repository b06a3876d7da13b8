#!/usr/bin/env python
"""Benchmark of the quantized decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload decode|matvec|attention]
                    [--prompt P] [--batch B]

Prints ONE JSON line (rank 0).  Workloads are synthetic and seeded (random-init weights of the named
shape; no checkpoint or dataset is read):

  decode  (default) Llama-3-8B-shaped model: 32 layers, hidden 4096, FFN 14336 SwiGLU, 32 Q / 8 KV heads,
          head_dim 128, RoPE theta 5e5, vocab 128256, weights ~ N(0, 0.02) quantized INT4 g128 with AWQ
          scales ~ U(0.5, 2), fp16 embeddings / lm_head, TurboQuant INT8 KV.  A prompt of P tokens is
          prefilled, then one step = one greedy decode step of the whole model at batch B; `value` is
          tokens/s of K steps replayed as CUDA graphs with the token fed back on the device; `e2e` is the
          same loop through decode_step() with the token coming from host memory and the logits going
          back to host memory every step.  With --gpus N the model is tensor-parallel over N ranks.
  matvec  one step = the four INT4 g128 projection launches of one decoder layer at batch 1
          (fused QKV 4096->6144, o 4096->4096, fused gate+up+SiLU 4096->2x14336, down 14336->4096),
          each step on a different weight copy out of a rotation larger than L2; value = GB/s.

  attention  TurboQuant INT8-KV decode attention alone at context --prompt and batch --batch (32 Q / 8 KV heads); GB/s of KV bytes.

`--impl reference` times the CPU restatement of the reference's own CPU path (the oracle) on the host
cores for the same workload, on a bounded sample.
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

GS = 128
L8 = dict(architecture="llama", hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
          num_key_value_heads=8, head_dim=128, vocab_size=128256, max_position_embeddings=8192, rms_norm_eps=1e-5,
          rope_theta=5e5, tie_word_embeddings=False)
Q06 = dict(architecture="qwen3", hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
           num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=8192, rms_norm_eps=1e-6,
           rope_theta=1e6, tie_word_embeddings=False)
MODELS = {"llama3_8b": (L8, True, "llama3_8b_shape_int4_g128_awq_tq8_decode"),      # (shape, AWQ scales, workload name)
          "qwen3_0p6b": (Q06, False, "qwen3_0p6b_shape_int4_g128_tq8_decode")}
# Llama-3-8B-shaped projections: (name, N, K, kind)
L8_SHAPES = [("qkv", 6144, 4096, "plain"), ("o", 4096, 4096, "plain"),
             ("gate_up", 14336, 4096, "ffn"), ("down", 4096, 14336, "plain")]
METRIC_DECODE = "decode tok/s (Llama-3-8B shape, INT4 g128 + AWQ weights, INT8 TurboQuant KV)"
METRIC_DECODE_Q = "decode tok/s (Qwen3-0.6B shape, INT4 g128 weights, INT8 TurboQuant KV)"
METRIC_MATVEC = "matvec HBM GB/s (INT4 g128 affine, Llama-3-8B projection shapes, batch 1)"
METRIC_ATTN = "TurboQuant INT8-KV decode attention HBM GB/s (32 Q / 8 KV heads, head_dim 128)"
# dram__bytes_read.sum + dram__bytes_write.sum from the ncu captures summarised under profiles/
PROJ_DRAM_BYTES = 62467840 + 17920          # matvec_v2_kernel<gate+up+SiLU>, one launch
TOKEN_KERNEL_DRAM_BYTES_PER_LAYER = (968957440 + 41039104) / 8   # dram read + write of the 8-layer ncu capture (profiles/decode_token_kernel_l8_shapes_ctx2k.md)


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
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.2)
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
        time.sleep(0.1)
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
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, no MEASURED_PEAKS.json beside this file)"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s (burst) of the roofline: the cuBLAS figure in MEASURED_PEAKS.json, else 1590."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path)).get("bf16_tflops", 1590.0))
    return 1590.0


# ----------------------------------------------------------------------------- synthetic weights on the GPU
def gpu_quantized(dev, N, K, gen, awq):
    import torch

    from ironmill_b200 import ops
    w = (torch.randn((N, K), generator=gen, device="cuda") * 0.02).half()
    packed, s, z = ops.quantize_affine(w, GS, 4, awq)
    return packed, s, z


def gpu_layer_copy(dev, seed):
    """One copy of the four projections, quantized ON the GPU with the library's own quantizer."""
    import torch

    from ironmill_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = {}
    for name, N, K, kind in L8_SHAPES:
        awq = (torch.rand(K, generator=g, device="cuda") * 1.5 + 0.5).half()
        mats = []
        for _ in range(2 if kind == "ffn" else 1):
            packed, s, z = gpu_quantized(dev, N, K, g, awq)
            mats.append(ops.AffineWeight(dev, packed, s, z, N, K, GS, 4, awq=awq))
        out[name] = mats
    return out


class SyntheticL8Provider:
    """WeightProvider of a random-init Llama-3-8B-shaped model: tensors are drawn with a seeded torch
    generator on the GPU, quantized by the library's GPU quantizer (bit-exact with the reference's CPU
    quantizer) and handed over as host arrays, like a bundle provider would."""

    def __init__(self, cfg, dev, seed=1234, awq=True):
        self.cfg, self.dev, self.seed, self.awq = cfg, dev, seed, awq

    def config(self):
        return self.cfg

    def has_tensor(self, name):
        return True

    def tensor(self, name):
        import zlib

        import torch

        from ironmill_b200.bundle import WeightTensor
        c = self.cfg
        g = torch.Generator(device="cuda").manual_seed(self.seed * 7919 + zlib.crc32(name.encode()))
        Hd, I, hd = c.hidden_size, c.intermediate_size, c.head_dim
        if name.endswith("layernorm.weight") or name == "model.norm.weight" or name.endswith("_norm.weight"):
            n = hd if "self_attn" in name else Hd
            return WeightTensor(np.ones(n, np.float16), (n,), "float16")
        if name in ("model.embed_tokens.weight", "lm_head.weight"):
            w = (torch.randn((c.vocab_size, Hd), generator=g, device="cuda") * 0.02).half()
            return WeightTensor(w.cpu().numpy(), (c.vocab_size, Hd), "float16")
        shapes = {"q_proj": (c.num_attention_heads * hd, Hd, "attn_in"), "k_proj": (c.num_key_value_heads * hd, Hd, "attn_in"),
                  "v_proj": (c.num_key_value_heads * hd, Hd, "attn_in"), "o_proj": (Hd, c.num_attention_heads * hd, "o_in"),
                  "gate_proj": (I, Hd, "ffn_in"), "up_proj": (I, Hd, "ffn_in"), "down_proj": (Hd, I, "down_in")}
        key = name.split(".")[-2]
        N, K, grp = shapes[key]
        layer = name.split(".")[2]
        ga = torch.Generator(device="cuda").manual_seed(self.seed * 104729 + zlib.crc32(f"{layer}.{grp}".encode()))
        awq = (torch.rand(K, generator=ga, device="cuda") * 1.5 + 0.5).half() if self.awq else None   # shared by projections with one input
        packed, s, z = gpu_quantized(self.dev, N, K, g, awq)
        return WeightTensor(packed.cpu().numpy(), (N, K), "uint8", s.cpu().numpy(), z.cpu().numpy(), 4, GS, 1,
                            None if awq is None else awq.cpu().numpy())


def time_dominant_kernel(dev, reps=5):
    """Average duration of the fused gate+up+SiLU matvec launch (the largest kernel of a decode step),
    CUDA events around a CUDA graph of launches that rotate over weight copies larger than L2."""
    import torch

    from ironmill_b200 import ops
    N, K = 14336, 4096
    ncopy = 6
    g = torch.Generator(device="cuda").manual_seed(5)
    awq = (torch.rand(K, generator=g, device="cuda") * 1.5 + 0.5).half()
    gates = [ops.AffineWeight(dev, *gpu_quantized(dev, N, K, g, awq), N, K, GS, 4, awq=awq) for _ in range(ncopy)]
    ups = [ops.AffineWeight(dev, *gpu_quantized(dev, N, K, g, awq), N, K, GS, 4, awq=awq) for _ in range(ncopy)]
    x = torch.randn((1, K), generator=g, device="cuda").half()
    y = torch.empty((1, N), dtype=torch.float16, device="cuda")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(ncopy):
            ops.ffn_gate_up_act(gates[i], ups[i], x, out=y)
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            for i in range(ncopy):
                ops.ffn_gate_up_act(gates[i], ups[i], x, out=y)
        graph.replay()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(reps):
            graph.replay()
        e1.record(s)
        s.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * ncopy)
    nbytes = shape_bytes("gate_up", N, K, "ffn")
    del gates, ups
    return us, nbytes, reps * ncopy


def run_decode(args, rank, world):
    import torch
    import torch.distributed as dist

    from ironmill_b200 import ops
    from ironmill_b200.bundle import ModelConfig
    from ironmill_b200.engine import CudaConfig, CudaInference

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        # NCCL carries only set-up, the logits gather and prefill-size all-reduces here: in-switch reduction buys nothing, and
        # every multi-GPU number of this repo was taken with it off (override by exporting NCCL_NVLS_ENABLE=1)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    dev = ops.Device(local)
    shape, with_awq, workload = MODELS[args.model]
    cfg = ModelConfig(**dict(shape, num_hidden_layers=args.layers or shape["num_hidden_layers"]))
    B, P, K, W = args.batch, args.prompt, args.steps, max(args.warmup, 3)
    e2e_steps = max(8, min(K, 64))
    max_seq = P + W + K + e2e_steps + 8
    eng = CudaInference(CudaConfig(max_seq_len=max_seq, max_batch=B, tp_world=world, tp_rank=rank, device=local))
    t0 = time.perf_counter()
    eng.load_weights(SyntheticL8Provider(cfg, dev, awq=with_awq))
    if world > 1:
        ids = [CudaInference.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        eng.tp_init(ids[0])
    load_s = time.perf_counter() - t0
    prompt = np.random.Generator(np.random.PCG64(11)).integers(0, cfg.vocab_size, P).astype(np.uint32)
    t0 = time.perf_counter()
    logits = eng.prefill(prompt)
    prefill_s = time.perf_counter() - t0
    first = np.full(B, int(logits.argmax()), dtype=np.uint32)
    if B > 1:   # every sequence of the batch gets the whole prompt in its own cache slot
        eng.reset()
        t0 = time.perf_counter()
        for _ in range(B):
            eng.add_sequence(prompt)
        prefill_s = (time.perf_counter() - t0) / B
    toks, _ = eng.decode_greedy(first, W)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()   # before the barrier: its start-up must not delay this rank inside the timed region
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    ctx0 = eng.seq_pos()
    toks, ms = eng.decode_greedy(toks[-1], K)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ctx_mid = ctx0 + K // 2

    # end to end: decode_step() per token, token from host memory, fp16 logits copied back and widened on the host
    tok = toks[-1].copy()
    eng.decode_step(tok if B > 1 else int(tok[0]))
    w0 = time.perf_counter()
    for _ in range(e2e_steps):
        lg = eng.decode_step(tok if B > 1 else int(tok[0]))
        tok = np.atleast_2d(lg).argmax(-1).astype(np.uint32)
    e2e_s = time.perf_counter() - w0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    prof = eng.profile_step(B)
    step_bytes = eng.step_bytes(ctx_mid, B)
    launches = eng.step_launches()
    # dominant kernel: the whole-token decode kernel when the engine uses it (batch 1, one GPU), else the largest projection launch
    tk = eng.token_kernel_profile(8) if (B == 1 and eng.token_kernel()) else None   # every rank: the kernels of a tensor-parallel model wait on one another
    dom_us, dom_bytes, _ = time_dominant_kernel(dev) if (rank == 0 and args.model == "llama3_8b") else (1.0, 0, 0)
    if rank != 0:
        return
    peak, peak_src = measured_peaks()
    tok_s = B * K / (ms * 1e-3)
    step_gbs = step_bytes / (ms / K * 1e-3) / 1e9
    proj = {"kernel": "matvec_v2_kernel<gate+up+SiLU, batch 1> 4096->2x14336 (largest projection, launched alone)",
            "achieved": round(dom_bytes / (dom_us * 1e-6) / 1e9, 1), "frac": round(dom_bytes / (dom_us * 1e-6) / 1e9 / peak, 4),
            "bytes_per_launch": dom_bytes, "us_per_launch": round(dom_us, 3),
            "timing": "CUDA events around a CUDA graph of launches rotating over 6 weight copies (702 MB > L2)"}
    if tk is not None:
        tk_ms, phases = tk
        head_bytes = (cfg.vocab_size // world) * cfg.hidden_size * 2 + 2 * cfg.hidden_size * 2 + (cfg.vocab_size // world) * 2   # this rank's lm_head rows + embedding row + logits
        tk_bytes = step_bytes - head_bytes
        roof = {"bound": "hbm", "kernel": "decode_token_kernel (all %d layers of one token: projections, RoPE + cache write, attention)" % cfg.num_hidden_layers,
                "achieved": round(tk_bytes / (tk_ms * 1e-3) / 1e9, 1), "peak": peak, "unit": "GB/s",
                "frac": round(tk_bytes / (tk_ms * 1e-3) / 1e9 / peak, 4), "peak_source": peak_src,
                "bytes_per_launch": tk_bytes, "us_per_launch": round(tk_ms * 1e3, 1),
                "traffic": int(TOKEN_KERNEL_DRAM_BYTES_PER_LAYER * cfg.num_hidden_layers) if world == 1 else None,
                "traffic_note": ("dram read+write per launch: ncu capture of an 8-layer model of the same shapes scaled by the layer count (profiles/)"
                                 if world == 1 else "no ncu capture of the tensor-parallel kernel (a multi-rank command is never profiled)"),
                "timing": "CUDA events around 8 back-to-back launches on the engine's stream; every launch streams all weights (> L2)",
                "phase_us_per_layer": {k: round(v, 2) for k, v in phases.items()},
                "largest_projection_alone": proj if args.model == "llama3_8b" else None}
    elif args.model == "llama3_8b" and B < 16:
        roof = dict(proj, bound="hbm", peak=peak, unit="GB/s", peak_source=peak_src, traffic=PROJ_DRAM_BYTES,
                    traffic_note="dram read+write of this launch from the ncu capture under profiles/")
    else:
        roof = {"bound": "hbm", "kernel": "whole step (graph of per-projection kernels; from 16 rows on the projections are tcgen05 GEMMs)",
                "achieved": round(step_gbs, 1), "peak": peak,
                "unit": "GB/s", "frac": round(step_gbs / peak, 4), "peak_source": peak_src, "traffic": None}
    roof["whole_step"] = {"bytes_per_step_per_gpu": step_bytes, "achieved_gbs_per_gpu": round(step_gbs, 1),
                          "frac_of_hbm_roofline": round(step_gbs / peak, 4),
                          "roofline_tok_s": round(B * peak * 1e9 / step_bytes, 1)}
    out = {
        "metric": METRIC_DECODE if args.model == "llama3_8b" else METRIC_DECODE_Q, "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(ms / K, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u4 codes x i24 activations (f32 fix-up), f16 lm_head, u8 KV codebook indices",
        "data": "synthetic",
        "config": decode_config(workload, cfg, B, P, world),
        "run": {"context_during_timing": [ctx0, ctx0 + K],
                "allreduce": (("inside the whole-token kernel: partial sums stored to every rank's mailbox over NVLink with tags, summed by the consuming phase, no barrier"
                               if (B == 1 and eng.token_kernel()) else "one-shot peer-memory kernel")
                              if eng.tp_peer_allreduce() else "nccl") if world > 1 else None,
                "bytes_per_step_per_gpu": step_bytes, "load_s": round(load_s, 1), "prefill_s_per_sequence": round(prefill_s, 3)},
        "roofline": roof,
        "e2e": {"value": round(B * e2e_steps / e2e_s, 2), "unit": "tok/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 2 * B * cfg.vocab_size, "steps": e2e_steps,
                "note": "InferenceEngine.decode_step per token: host token in, fp16 logits to pinned host memory, widened to f32"},
        "gpu_launches": launches * K,
        "launches_per_step": launches,
        "step_profile_ms": {k: round(v, 4) for k, v in prof.items()},
        "step_profile_note": "per-category timing of the launch-per-kernel schedule run eagerly (the schedule used for batch > 1); "
                             "the timed steps above run the whole-token kernel when roofline.kernel says so",
        "clocks": clocks,
    }
    if world == 1:
        out["cpu_baseline"] = cpu_decode_baseline(args.model, B, P, budget_s=20.0, min_steps=3)
    print(json.dumps(out))


def decode_config(workload, cfg, B, P, world):
    """The workload as both arms name it (the same keys and values in the GPU arm and in --impl reference)."""
    return {"workload": workload, "batch": B, "prompt_tokens": P, "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
            "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size, "parallelism": f"tp{world}" if world > 1 else "single",
            "l2_policy": "inputs larger than L2: every step streams all of the rank's weights and its KV cache"}


def time_projection(dev, N, K, kind, B, bits, awq_on=True, reps=4):
    """Microseconds per launch of one projection at batch B (CUDA events around a CUDA graph that rotates over enough
    weight copies to exceed L2): batch <= 4 runs the matvec kernels (one launch), batch >= 16 the tcgen05 GEMM (gate and
    up as two GEMMs + the SiLU kernel).  Returns (us, algorithmic bytes, flops, launches per call)."""
    import torch

    from ironmill_b200 import ops
    nmat = 2 if kind == "ffn" else 1
    wbytes = nmat * (N * K * bits // 8 + 4 * N * (K // GS))
    ncopy = max(3, min(96, int(170e6 // wbytes) + 1))
    g = torch.Generator(device="cuda").manual_seed(N + K + B)
    awq = (torch.rand(K, generator=g, device="cuda") * 1.5 + 0.5).half() if awq_on else None
    copies = []
    for _ in range(ncopy):
        mats = []
        for _ in range(nmat):
            w = (torch.randn((N, K), generator=g, device="cuda") * 0.02).half()
            packed, sc, zp = ops.quantize_affine(w, GS, bits, awq)
            mats.append(ops.AffineWeight(dev, packed, sc, zp, N, K, GS, bits, awq=awq))
        copies.append(mats)
    x = torch.randn((B, K), generator=g, device="cuda").half()
    y = torch.empty((B, N), dtype=torch.float16, device="cuda")
    y2 = torch.empty((B, N), dtype=torch.float16, device="cuda")
    scratch = torch.empty((B, K), dtype=torch.float16, device="cuda")
    gemm = B >= 16 and bits == 4

    def call(i):
        m = copies[i % ncopy]
        if gemm:
            ops.matmul_affine(m[0], x, out=y, scratch=scratch)
            if kind == "ffn":
                ops.matmul_affine(m[1], x, out=y2, scratch=scratch)
                ops.silu_mul(y, y2, out=y)
        elif kind == "ffn":
            ops.ffn_gate_up_act(m[0], m[1], x, out=y)
        else:
            ops.matvec_affine(m[0], x, out=y)

    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for i in range(ncopy):   # every copy once outside the capture: the paired gate/up tile stream is built on first use
            call(i)
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for i in range(ncopy):
                call(i)
        graph.replay()
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(reps):
            graph.replay()
        e1.record(st)
        st.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * ncopy)
    nbytes = wbytes + B * K * 2 + B * N * 2 + (K * 2 if awq_on else 0)
    del copies
    torch.cuda.empty_cache()
    return us, nbytes, 2.0 * nmat * B * N * K


def run_matvec(args, rank, world):
    """The single-kernel sweep: headline = the four INT4 g128 projection launches of one decoder layer at batch 1; `sweep`
    lists every projection shape at batch 1 / 4 / 16 / 64, the shards a rank holds under 2 / 4 / 8-way tensor
    parallelism (column split N / G for QKV and gate+up, row split K / G for o and down) and the INT8 form."""
    import torch

    from ironmill_b200 import ops
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = ops.Device(local)
    ncopies = 4   # 4 x 116 MB of weights > 126 MB of L2: no step finds its weights cached
    copies = [gpu_layer_copy(dev, 100 + i) for i in range(ncopies)]
    g = torch.Generator(device="cuda").manual_seed(7)
    xs = {K: torch.randn((1, K), generator=g, device="cuda").half() for K in (4096, 14336)}
    ys = {name: torch.empty((1, N), dtype=torch.float16, device="cuda") for name, N, K, kind in L8_SHAPES}
    step_bytes = sum(shape_bytes(*s) for s in L8_SHAPES)

    def step(i):
        cp = copies[i % ncopies]
        for name, N, K, kind in L8_SHAPES:
            if kind == "ffn":
                ops.ffn_gate_up_act(cp[name][0], cp[name][1], xs[K], out=ys[name])
            else:
                ops.matvec_affine(cp[name][0], xs[K], out=ys[name])

    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(max(args.warmup, ncopies)):
            step(i)
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            for i in range(ncopies):
                step(i)
        graph.replay()
        s.synchronize()
        reps = max(1, args.steps // ncopies)
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(reps):
            graph.replay()
        e1.record(s)
        s.synchronize()
        clocks = sampler.stop()
    steps = reps * ncopies
    ms = e0.elapsed_time(e1)
    xh = {K: np.random.default_rng(1).standard_normal((1, K)).astype(np.float16) for K in (4096, 14336)}
    plain = [sh for sh in L8_SHAPES if sh[3] == "plain"]
    for name, N, K, kind in plain:
        ops.matvec_affine_host(copies[0][name][0], xh[K])
    w0 = time.perf_counter()
    for i in range(20):
        for name, N, K, kind in plain:
            ops.matvec_affine_host(copies[i % ncopies][name][0], xh[K])
    e2e_s = time.perf_counter() - w0
    del copies
    torch.cuda.empty_cache()
    dom_us, dom_bytes, _ = time_dominant_kernel(dev)
    peak, peak_src = measured_peaks()
    tpeak = measured_tensor_peak()
    sweep = []
    cases = [(n, N, K, kind, B, 4, 1) for n, N, K, kind in L8_SHAPES for B in (1, 4, 16, 64)]
    cases += [(n, N, K, kind, B, 4, 1) for n, N, K, kind in L8_SHAPES for B in (256, 2048)]   # prefill chunks: the tensor-core GEMM
    cases += [(n, N, K, kind, 1, 8, 1) for n, N, K, kind in L8_SHAPES]
    for G in (2, 4, 8):   # what one of G ranks holds
        cases += [(n, N // G if n in ("qkv", "gate_up") else N, K if n in ("qkv", "gate_up") else K // G, kind, 1, 4, G) for n, N, K, kind in L8_SHAPES]
    if not args.sweep:
        cases = []
    for n, N, K, kind, B, bits, G in cases:
        us, nb, fl = time_projection(dev, N, K, kind, B, bits)
        row = {"shape": n, "N": N, "K": K, "batch": B, "bits": bits, "tp_shard_of": G, "us": round(us, 2),
               "GBps": round(nb / us / 1e3, 1), "frac_hbm": round(nb / us / 1e3 / peak, 3)}
        if B >= 16 and bits == 4:
            row["TFLOPs"] = round(fl / us / 1e6, 1)
            row["frac_tensor"] = round(fl / us / 1e6 / tpeak, 4)
            row["kernel"] = "gemm_int4_tc_kernel (tcgen05)"
        sweep.append(row)
    out = {"metric": METRIC_MATVEC, "value": round(step_bytes * steps / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "n_gpus": 1,
           "steps": steps, "warmup": args.warmup, "ms_per_step": round(ms / steps, 5), "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "u4 codes x i24 activations, f32 fix-up", "data": "synthetic",
           "config": {"workload": "int4_g128_matvec_sweep_llama3_8b_shapes_b1_awq", "shapes": [[n, N, K] for n, N, K, _ in L8_SHAPES],
                      "l2_policy": f"rotation over {ncopies} weight copies ({ncopies * step_bytes >> 20} MiB) larger than L2"},
           "roofline": {"bound": "hbm", "kernel": "matvec_v2_kernel<gate+up+SiLU, batch 1> 4096->2x14336",
                        "achieved": round(dom_bytes / (dom_us * 1e-6) / 1e9, 1), "peak": peak, "unit": "GB/s",
                        "frac": round(dom_bytes / (dom_us * 1e-6) / 1e9 / peak, 4), "peak_source": peak_src, "traffic": PROJ_DRAM_BYTES,
                        "bytes_per_launch": dom_bytes, "us_per_launch": round(dom_us, 3)},
           "e2e": {"value": round(sum(shape_bytes(*sh) for sh in plain) * 20 / e2e_s / 1e9, 3), "unit": "GB/s",
                   "h2d_bytes_per_step": sum(K * 2 for _, N, K, _ in plain), "d2h_bytes_per_step": sum(N * 2 for _, N, K, _ in plain)},
           "gpu_launches": 4 * steps, "clocks": clocks, "sweep": sweep, "cpu_baseline": cpu_matvec_baseline(3.0)}
    print(json.dumps(out))


def run_attention(args, rank, world):
    """TurboQuant INT8 KV decode attention alone (split attention + reduction), one step = one decode token of `batch`
    sequences at context --prompt: value = KV bytes read (codes + scales + residual norms) / time.  The cache holds
    random codes and positive scales (the kernel's work does not depend on the values); rotating over enough cache
    copies keeps every step's KV out of L2."""
    import torch

    from ironmill_b200 import ops
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = ops.Device(local)
    nh, nkv, hd, ctx, B, bits = 32, 8, 128, args.prompt, args.batch, args.kv_bits
    signs, qjl = ops.tq_generate(hd, 42)
    tq = ops.TurboQuant(dev, hd, bits, signs, qjl) if bits != 16 else None
    kv_bytes = B * nkv * ctx * (2 * hd * bits // 8 + (12 if bits != 16 else 0))
    ncopy = max(2, int(400e6 // kv_bytes) + 1)
    g = torch.Generator(device="cuda").manual_seed(3)
    caches = []
    for _ in range(ncopy):
        if bits == 16:   # fp16 rows (TurboQuant off)
            caches.append(((torch.randn((B, nkv, ctx, hd), generator=g, device="cuda") * 0.5).half(),
                           torch.randn((B, nkv, ctx, hd), generator=g, device="cuda").half()))
            continue
        kc = torch.randint(0, 256, (B, nkv, ctx, hd * bits // 8), generator=g, device="cuda", dtype=torch.uint8)
        vc = torch.randint(0, 256, (B, nkv, ctx, hd * bits // 8), generator=g, device="cuda", dtype=torch.uint8)
        ks = torch.rand((B, nkv, ctx), generator=g, device="cuda") + 0.5
        vs = torch.rand((B, nkv, ctx), generator=g, device="cuda") + 0.5
        kr = torch.rand((B, nkv, ctx), generator=g, device="cuda") * 0.1
        caches.append((kc, vc, ks, vs, kr))
    q = torch.randn((B, nh, hd), generator=g, device="cuda").half()
    scale = 1.0 / np.sqrt(hd)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")

    def step(i):
        if bits == 16:
            k16, v16 = caches[i % ncopy]
            return ops.sdpa_f16(dev, q, k16, v16, scale, nh, nkv, ctx, 0, nseq=B, pos_dev=pos)
        kc, vc, ks, vs, kr = caches[i % ncopy]
        return tq.attention(q, kc, vc, ks, vs, kr, scale, nh, nkv, ctx, ctx - 1, nseq=B)

    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(max(args.warmup, 3)):
            step(i)
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            for i in range(ncopy):
                step(i)
        graph.replay()
        s.synchronize()
        reps = max(1, args.steps // ncopy)
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(reps):
            graph.replay()
        e1.record(s)
        s.synchronize()
        clocks = sampler.stop()
    steps = reps * ncopy
    ms = e0.elapsed_time(e1)
    peak, peak_src = measured_peaks()
    gbs = kv_bytes * steps / (ms * 1e-3) / 1e9
    qh = q.cpu()
    w0 = time.perf_counter()
    for i in range(8):
        step(i).cpu()
        q.copy_(qh, non_blocking=False)
    e2e_s = time.perf_counter() - w0
    metric = METRIC_ATTN if bits == 8 else METRIC_ATTN.replace("TurboQuant INT8-KV", "TurboQuant INT4-KV" if bits == 4 else "fp16-KV")
    out = {"metric": metric, "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
           "ms_per_step": round(ms / steps, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "u8 codebook indices, f32 accumulation" if bits != 16 else "f16 rows, f32 accumulation", "data": "synthetic",
           "config": {"workload": {8: "turboquant_int8_kv_decode_attention", 4: "turboquant_int4_kv_decode_attention",
                                   16: "fp16_kv_decode_attention"}[bits], "context": ctx, "batch": B, "q_heads": nh, "kv_heads": nkv,
                      "l2_policy": f"rotation over {ncopy} cache copies ({ncopy * kv_bytes >> 20} MiB) larger than L2"},
           "roofline": {"bound": "hbm", "kernel": "tq_attention_tc_kernel<4> + tq_reduce_kernel" if bits != 16 else "sdpa16_kernel<4> + sdpa16_reduce_kernel",
                        "achieved": round(gbs, 1), "peak": peak,
                        "unit": "GB/s", "frac": round(gbs / peak, 4), "peak_source": peak_src, "bytes_per_launch": kv_bytes,
                        "us_per_launch": round(ms / steps * 1e3, 2), "traffic": None},
           "e2e": {"value": round(kv_bytes * 8 / e2e_s / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": B * nh * hd * 2,
                   "d2h_bytes_per_step": B * nh * hd * 2},
           "gpu_launches": 2 * steps, "clocks": clocks}
    print(json.dumps(out))


# ----------------------------------------------------------------------------- CPU arm (the oracle, timed)
def cpu_matvec_baseline(seconds):
    from oracle import oracle as orc
    threads = host_threads(orc)
    rng = np.random.default_rng(0)
    N = K = 4096
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    x = rng.standard_normal((1, K)).astype(np.float16)
    t0 = time.perf_counter()
    codes, scales, zps = orc.quantize_groups(w, GS, 4, threads=threads)
    packed = orc.pack_int4(codes)
    tq = time.perf_counter() - t0
    s16, z16 = orc.f32_to_f16(scales), orc.f32_to_f16(zps)
    reps, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        orc.matvec_affine(packed, s16, z16, x, N, K, GS, 4, threads=threads)
        reps += 1
    tm = (time.perf_counter() - t0) / reps
    return {"value": round(matvec_bytes(N, K, awq=False) / tm / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"4096x4096 INT4 g128 matvec, batch 1, {reps} repetitions, OpenMP {threads} threads; quantize+pack {tq * 1e3:.0f} ms",
            "quantize_ms": round(tq * 1e3, 1), "matvec_ms": round(tm * 1e3, 3)}


def cpu_decode_baseline(model, B, P, budget_s, min_steps):
    """The CPU restatement of the reference's path (the oracle, OpenMP on every core this process may use) running REAL
    decode tokens of the named model at context P, batch 1 per token: per layer the fused QKV matvec, RoPE (with QK-norm
    where the model has it), the TurboQuant write of K and V, TurboQuant attention over P cached positions, o,
    residual + RMSNorm, gate/up + SiLU, down, residual add; then the final norm, the whole fp16 lm_head and the greedy
    pick.  Bounded sample: the token runs all its layers over `sets` distinct sets of layer weights taken in turn
    (every set is far larger than the CPU caches), caches hold random codes, and as many whole tokens are timed as fit
    the budget (at least min_steps)."""
    from oracle import oracle as orc
    shape, with_awq, _ = MODELS[model]
    Hd, I, hd, nh, nkv, L, V = (shape[k] for k in ("hidden_size", "intermediate_size", "head_dim", "num_attention_heads",
                                                    "num_key_value_heads", "num_hidden_layers", "vocab_size"))
    threads = host_threads(orc)
    rng = np.random.default_rng(0)
    sets, nsets = [], 2
    max_seq = P + 64
    tq0 = time.perf_counter()
    tqc = orc.TqConstants(hd, 8, seed=42)
    for _ in range(nsets):
        d = {}
        for name, N, K in (("qkv", (nh + 2 * nkv) * hd, Hd), ("o", Hd, nh * hd), ("gate", I, Hd), ("up", I, Hd), ("down", Hd, I)):
            w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02).astype(np.float16)
            awq = rng.uniform(0.5, 2.0, K).astype(np.float16) if with_awq else None
            codes, sc, zp = orc.quantize_groups(w, GS, 4, awq=awq, threads=threads)
            d[name] = (orc.pack_int4(codes), orc.f32_to_f16(sc), orc.f32_to_f16(zp), awq, N, K)
        d["kc"] = rng.integers(0, 256, (nkv, max_seq, hd), dtype=np.uint8)
        d["vc"] = rng.integers(0, 256, (nkv, max_seq, hd), dtype=np.uint8)
        d["ks"], d["vs"] = (rng.random((nkv, max_seq), dtype=np.float32) + 0.5 for _ in range(2))
        d["kr"] = rng.random((nkv, max_seq), dtype=np.float32) * 0.1
        d["g1"], d["g2"] = np.ones(Hd, np.float16), np.ones(Hd, np.float16)
        d["qn"], d["kn"] = np.ones(hd, np.float16), np.ones(hd, np.float16)
        sets.append(d)
    quant_s = time.perf_counter() - tq0
    lm = (rng.standard_normal((V, Hd), dtype=np.float32) * 0.02).astype(np.float16)
    embed_row = (rng.standard_normal((1, Hd), dtype=np.float32) * 0.02).astype(np.float16)
    cos, sin = orc.rope_table(hd, max_seq, shape["rope_theta"])
    eps, scale = shape["rms_norm_eps"], 1.0 / np.sqrt(hd)
    qk_norm = shape["architecture"] == "qwen3"

    def mv(m, x):
        return orc.matvec_affine(m[0], m[1], m[2], x, m[4], m[5], GS, 4, awq=m[3], threads=threads)

    def token(pos):
        hidden = embed_row
        normed = orc.rms_norm(hidden, sets[0]["g1"], eps)
        for l in range(L):
            d = sets[l % nsets]
            qkv = mv(d["qkv"], normed)
            q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], np.ascontiguousarray(qkv[:, (nh + nkv) * hd:])
            if qk_norm:
                q, k = orc.qk_norm_rope(q, k, d["qn"], d["kn"], cos, sin, nh, nkv, hd, pos, eps)
            else:
                q, k = orc.rope(q, cos, sin, nh, hd, pos), orc.rope(k, cos, sin, nkv, hd, pos)
            orc.tq_encode(k, tqc, True, d["kc"], d["ks"], d["kr"], nkv, max_seq, pos)
            orc.tq_encode(v, tqc, False, d["vc"], d["vs"], None, nkv, max_seq, pos)
            attn = orc.tq_attention(q, d["kc"], d["vc"], tqc, d["ks"], d["vs"], d["kr"], scale, nh, nkv, max_seq, pos,
                                    num_splits=max(2, min(-(-(pos + 1) // 256), 256)) if pos + 1 >= 256 else 0).reshape(1, nh * hd)
            o = mv(d["o"], attn)
            normed, resid = orc.fused_residual_rms_norm(hidden, o, d["g2"], eps)
            g, u = d["gate"], d["up"]
            act = orc.ffn_gate_up_act(g[0], g[1], g[2], u[0], u[1], u[2], normed, I, Hd, GS, 4, awq=g[3], threads=threads)
            hidden = orc.residual_add(resid, mv(d["down"], act))
            normed = orc.rms_norm(hidden, d["g1"], eps)
        logits = orc.matvec_f16(lm, normed, threads=threads)
        return orc.argmax(logits.astype(np.float32))

    token(P)   # warm-up (page faults, OpenMP team)
    times = []
    while len(times) < min_steps or (sum(times) < budget_s and len(times) < 64):
        t0 = time.perf_counter()
        for b in range(B):
            token(P + 1 + len(times) % 32)
        times.append(time.perf_counter() - t0)
    step_s = float(np.median(times))
    return {"value": round(B / step_s, 4), "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{len(times)} whole decode step(s) of batch {B} at context {P} timed (median), every layer's projections, RoPE, TurboQuant write "
                      f"and attention, norms, the full lm_head and the greedy pick; the {L} layers take {nsets} distinct weight sets in turn; "
                      f"OpenMP {threads} threads; quantize+pack of the {nsets} sets took {quant_s:.1f} s",
            "steps_timed": len(times), "ms_per_step": round(step_s * 1e3, 1), "quantize_s": round(quant_s, 2)}


def host_threads(orc):
    """Threads for the CPU arm: all the cores this process may run on.  torchrun exports OMP_NUM_THREADS=1 to its workers,
    which would otherwise make the oracle's OpenMP loops single-threaded there."""
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    return max(int(orc.max_threads()), avail)


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU path as restated in oracle/ (kind "port": the reference itself is Rust + Metal
    and cannot be built here), on the host cores of rank 0, on the same workload and config as the GPU arm.  `steps` is
    the number of whole steps actually timed (bounded so that the run ends within a few minutes)."""
    if rank != 0:
        return
    t0 = time.perf_counter()
    if args.workload == "matvec":
        cb = cpu_matvec_baseline(8.0)
        out = {"impl": "reference", "metric": METRIC_MATVEC, "value": cb["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": cb["matvec_ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
               "dtype": "f32", "data": "synthetic",
               "config": {"workload": "int4_g128_matvec_sweep_llama3_8b_shapes_b1_awq", "shapes": [[n, N, K] for n, N, K, _ in L8_SHAPES]},
               "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(out))
        return
    from ironmill_b200.bundle import ModelConfig
    shape, _, workload = MODELS[args.model]
    cfg = ModelConfig(**dict(shape, num_hidden_layers=args.layers or shape["num_hidden_layers"]))
    budget = 60.0 if args.steps >= 8 else 20.0
    cb = cpu_decode_baseline(args.model, args.batch, args.prompt, budget_s=budget, min_steps=max(1, min(args.steps, 3)))
    out = {"impl": "reference", "metric": METRIC_DECODE if args.model == "llama3_8b" else METRIC_DECODE_Q, "value": cb["value"],
           "unit": "tok/s", "n_gpus": world, "steps": cb["steps_timed"], "warmup": 1, "ms_per_step": cb["ms_per_step"],
           "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": decode_config(workload, cfg, args.batch, args.prompt, world),
           "run": {"wall_s": round(time.perf_counter() - t0, 1), "steps_requested": args.steps,
                   "note": "whole decode steps on the host cores of rank 0; the tensor-parallel layout does not apply to the CPU arm"},
           "cpu_baseline": cb,
           "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "matvec", "attention"])
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="decoder layers of the synthetic model (0 = the named model's; fewer only for profiler captures)")
    ap.add_argument("--sweep", type=int, default=1, help="matvec workload: 1 = also time every shape at batch 1/4/16/64, INT8 and the tensor-parallel shards")
    ap.add_argument("--kv-bits", type=int, default=8, choices=[4, 8, 16], help="attention workload: TurboQuant bits, or 16 = fp16 KV cache")
    ap.add_argument("--model", default="llama3_8b", choices=sorted(MODELS), help="decode workload shape (the default is the headline configuration)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload == "matvec":
        run_matvec(args, rank, world)
    elif args.workload == "attention":
        run_attention(args, rank, world)
    else:
        run_decode(args, rank, world)
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        sys.stdout.flush()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
