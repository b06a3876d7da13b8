"""INT4 g128 GEMM on the tcgen05 tensor cores against the CPU oracle's matmul
(C[m,n] = sum_k f16(A[m,k]/awq[k]) * f16((q-z)s), f32 accumulation, fp16 result)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

# tolerance: same fp16 operands, f32 accumulation in a different order, one fp16 rounding of the result
TOL = 2e-3


@pytest.fixture(scope="module")
def dev():
    from ironmill_b200 import ops
    return ops.Device(0)


def _check(dev, qw, M, seed=0):
    from ironmill_b200 import ops
    x = (H.rng_for("gemm-x", seed).standard_normal((M, qw.K))).astype(np.float16)
    y = ops.matmul_affine(qw.gpu(dev), torch.from_numpy(x).cuda()).cpu().numpy()
    ref = orc.matmul_affine(qw.packed, qw.scales_f16, qw.zps_f16, x, qw.N, qw.K, 128, 4, awq=qw.awq, threads=8)
    err = H.rel_err(y, ref)
    assert err <= TOL, (qw.N, qw.K, M, err)
    return y, ref


@pytest.mark.parametrize("N,K,M", [(128, 128, 16), (256, 512, 32), (384, 1024, 70), (128, 256, 200), (1024, 1024, 129), (640, 384, 1)])
def test_shapes_and_token_tails(dev, N, K, M):
    _check(dev, H.QWeight(N, K, seed=N + M, name="g"), M)


@pytest.mark.parametrize("N,K,M", [(512, 2048, 16), (512, 2048, 64), (384, 1792, 33), (1024, 14336, 16), (200, 1024, 7)])
def test_k_split_for_few_tokens(dev, N, K, M):
    # at most 64 tokens against few 128-row tiles: the grid is cut along K (four slices here; an uneven last slice at
    # K = 1792 = 14 groups; ragged rows at N = 200), the f32 slices are added in order and rounded once
    _check(dev, H.QWeight(N, K, awq=True, seed=N + K + M, name="gk"), M)


@pytest.mark.parametrize("N,K,M", [(256, 512, 32), (384, 1024, 70), (1024, 1024, 129), (512, 2048, 16), (200, 512, 300)])
def test_int8_weights(dev, N, K, M):
    # superblock_matmul_int8 (affine_matmul.metal:155-290): byte codes through the same tensor-core kernel
    qw = H.QWeight(N, K, bits=8, awq=True, seed=N + K + M, name="g8")
    from ironmill_b200 import ops
    x = (H.rng_for("gemm-x8", M).standard_normal((M, K))).astype(np.float16)
    y = ops.matmul_affine(qw.gpu(dev), torch.from_numpy(x).cuda()).cpu().numpy()
    ref = orc.matmul_affine(qw.packed, qw.scales_f16, qw.zps_f16, x, N, K, 128, 8, awq=qw.awq, threads=8)
    assert H.rel_err(y, ref) <= TOL, (N, K, M)


def test_many_token_tiles_of_256(dev):
    # 19 token tiles x 8 row tiles: the 256-token tile (chosen once the grid covers the GPU), a ragged last token tile
    _check(dev, H.QWeight(1024, 512, awq=True, seed=77, name="gt"), 4700)


def test_awq_and_ragged_rows(dev):
    # N not a multiple of the 128-row CTA tile: the last CTA's spare rows are masked
    _check(dev, H.QWeight(200, 512, awq=True, seed=3, name="ga"), 48)


def test_llama_projection_shape(dev):
    _check(dev, H.QWeight(4096, 4096, awq=True, seed=5, name="gl"), 256)


def test_unusual_zero_points_take_the_f32_path(dev):
    # zero points that are not small integers (possible in a bundle written by another quantiser)
    qw = H.QWeight(256, 256, seed=9, name="gz")
    qw.zps = qw.zps.copy()
    qw.zps[::3] += 0.5
    qw.zps[1::7] = 3000.0
    qw.zps_f16 = orc.f32_to_f16(qw.zps)
    _check(dev, qw, 40)


def test_matches_the_matvec_kernel_rows(dev):
    # the same weight through the decode matvec (24-bit integer activations) and the GEMM: both within their tolerance of the oracle
    from ironmill_b200 import ops
    qw = H.QWeight(512, 1024, awq=True, seed=11, name="gm")
    w = qw.gpu(dev)
    x = torch.from_numpy(H.rng_for("gm-x").standard_normal((20, 1024)).astype(np.float16)).cuda()
    a = ops.matmul_affine(w, x).cpu().numpy().astype(np.float64)
    b = ops.matvec_affine(w, x).cpu().numpy().astype(np.float64)
    assert np.abs(a - b).max() / np.abs(b).max() <= 4e-3
