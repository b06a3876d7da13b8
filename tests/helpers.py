"""Seeded synthetic inputs shared by the tests (shapes and distributions of the decode configs)."""
import numpy as np

from oracle import oracle as orc


def rng_for(name: str, seed: int = 0):
    import zlib
    return np.random.Generator(np.random.PCG64(seed * 1000003 + zlib.crc32(name.encode())))


def make_weight(N, K, seed=0, name="w", std=0.02):
    return (rng_for(name, seed).standard_normal((N, K)) * std).astype(np.float16)


def make_awq(K, seed=0, name="awq"):
    return rng_for(name, seed).uniform(0.5, 2.0, K).astype(np.float16)


def make_x(B, K, seed=0, name="x"):
    return rng_for(name, seed).standard_normal((B, K)).astype(np.float16)


class QWeight:
    """A weight quantized by the CPU oracle: packed codes, f32 and fp16 params."""

    def __init__(self, N, K, bits=4, gs=128, awq=False, seed=0, name="w", threads=8, awq_vec=None):
        self.N, self.K, self.bits, self.gs = N, K, bits, gs
        self.w = make_weight(N, K, seed, name)
        self.awq = awq_vec if awq_vec is not None else (make_awq(K, seed, name + ".awq") if awq else None)
        self.codes, self.scales, self.zps = orc.quantize_groups(self.w, gs, bits, awq=self.awq, threads=threads)
        self.packed = orc.pack_int4(self.codes) if bits == 4 else self.codes.reshape(-1).copy()
        self.scales_f16 = orc.f32_to_f16(self.scales)
        self.zps_f16 = orc.f32_to_f16(self.zps)

    def gpu(self, dev):
        from ironmill_b200 import ops
        return ops.AffineWeight(dev, self.packed, self.scales, self.zps, self.N, self.K, self.gs, self.bits, awq=self.awq)


def rel_err(y, ref):
    """Max error relative to the largest reference magnitude (fp16 outputs)."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))
