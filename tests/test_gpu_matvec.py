"""Matvec family through the C ABI against the CPU oracle.

Tolerance: max |y - y_ref| <= 1e-2 * max |y_ref| (the stated gate for matvec outputs, fp16)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 1e-2


@pytest.fixture(scope="module")
def dev():
    from ironmill_b200 import ops
    return ops.Device(0)


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("N,K", [(8, 128), (33, 256), (64, 1024), (256, 3072), (130, 1792), (512, 4096)])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("awq", [False, True])
@pytest.mark.parametrize("B", [1, 2, 3, 4, 7])
def test_matvec_small(dev, N, K, bits, awq, B):
    from ironmill_b200 import ops
    qw = H.QWeight(N, K, bits=bits, awq=awq, seed=N + K)
    x = H.make_x(B, K, seed=B)
    ref = orc.matvec_affine(qw.packed, qw.scales_f16, qw.zps_f16, x, N, K, 128, bits, awq=qw.awq, threads=8)
    y = ops.matvec_affine(qw.gpu(dev), _cuda(x)).cpu().numpy()
    assert H.rel_err(y, ref) <= TOL
    # tighter: the kernel is far more accurate than the gate; catches layout slips
    assert H.rel_err(y, ref) <= 2e-3


@pytest.mark.parametrize("N,K,gs", [(5, 96, 32), (9, 200, 64), (3, 130, 128), (16, 512, 256), (4, 64, 128)])
@pytest.mark.parametrize("bits", [4, 8])
def test_matvec_other_group_sizes_and_ragged_k(dev, N, K, gs, bits):
    from ironmill_b200 import ops
    qw = H.QWeight(N, K, bits=bits, gs=gs, awq=True, seed=7)
    x = H.make_x(2, K, seed=1)
    ref = orc.matvec_affine(qw.packed, qw.scales_f16, qw.zps_f16, x, N, K, gs, bits, awq=qw.awq)
    y = ops.matvec_affine(qw.gpu(dev), _cuda(x)).cpu().numpy()
    assert H.rel_err(y, ref) <= 2e-3


def test_config1_cpu_reference_case(dev):
    """W [4096,4096] ~ N(0,0.02), INT4 g128, x ~ N(0,1), batch 1 (the CPU-runnable config)."""
    from ironmill_b200 import ops
    qw = H.QWeight(4096, 4096, seed=11)
    x = H.make_x(1, 4096, seed=11)
    ref = orc.matvec_affine(qw.packed, qw.scales_f16, qw.zps_f16, x, 4096, 4096, 128, 4, threads=8)
    w = qw.gpu(dev)
    y = ops.matvec_affine(w, _cuda(x)).cpu().numpy()
    assert H.rel_err(y, ref) <= TOL
    # host-buffer form of the same call
    y2 = ops.matvec_affine_host(w, x)
    assert (y2 == y).all()
    # dequant helper: bit-exact f16((q - z) * s)
    deq = w.dequant().cpu().numpy()
    ref_deq = orc.dequant_affine(qw.packed, qw.scales_f16, qw.zps_f16, (4096, 4096), 4, group_size=128)
    assert (deq.view(np.uint16) == ref_deq.view(np.uint16)).all()


@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 14336)])
@pytest.mark.parametrize("B", [1, 4])
def test_llama_projection_shapes(dev, N, K, B):
    from ironmill_b200 import ops
    qw = H.QWeight(N, K, awq=True, seed=5)
    x = H.make_x(B, K, seed=2)
    ref = orc.matvec_affine(qw.packed, qw.scales_f16, qw.zps_f16, x, N, K, 128, 4, awq=qw.awq, threads=8)
    y = ops.matvec_affine(qw.gpu(dev), _cuda(x)).cpu().numpy()
    assert H.rel_err(y, ref) <= 2e-3


def test_deterministic(dev):
    from ironmill_b200 import ops
    qw = H.QWeight(4096, 4096, seed=3)
    w = qw.gpu(dev)
    x = _cuda(H.make_x(4, 4096))
    a = ops.matvec_affine(w, x).clone()
    b = ops.matvec_affine(w, x)
    assert torch.equal(a, b)


@pytest.mark.parametrize("I,K", [(64, 128), (200, 1024), (3072, 1024), (1024, 4096)])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("B", [1, 3])
def test_ffn_gate_up_act(dev, I, K, bits, B):
    from ironmill_b200 import ops
    g = H.QWeight(I, K, bits=bits, awq=True, seed=21, name="gate")
    u = H.QWeight(I, K, bits=bits, seed=21, name="up", awq_vec=g.awq)   # gate and up share the input scales
    x = H.make_x(B, K, seed=4)
    ref = orc.ffn_gate_up_act(g.packed, g.scales_f16, g.zps_f16, u.packed, u.scales_f16, u.zps_f16, x, I, K, 128, bits,
                              awq=g.awq, threads=8)
    y = ops.ffn_gate_up_act(g.gpu(dev), u.gpu(dev), _cuda(x)).cpu().numpy()
    assert H.rel_err(y, ref) <= 3e-3


@pytest.mark.parametrize("N,K", [(64, 128), (2048, 1024), (300, 4096)])
@pytest.mark.parametrize("awq", [False, True])
@pytest.mark.parametrize("B", [1, 2])
def test_fused_residual_norm_matvec(dev, N, K, awq, B):
    from ironmill_b200 import ops
    qw = H.QWeight(N, K, awq=awq, seed=31)
    a = H.make_x(B, K, seed=5, name="a")
    b = H.make_x(B, K, seed=5, name="b")
    gamma = (1.0 + 0.1 * H.rng_for("gamma").standard_normal(K)).astype(np.float16)
    ry, rres, rnrm = orc.fused_residual_norm_matvec(a, b, gamma, qw.packed, qw.scales_f16, qw.zps_f16, 1e-6, N, K, 128, 4,
                                                    awq=qw.awq, threads=8)
    y, res, nrm = ops.fused_residual_norm_matvec(qw.gpu(dev), _cuda(a), _cuda(b), _cuda(gamma), 1e-6)
    assert H.rel_err(y.cpu().numpy(), ry) <= 3e-3
    assert (res.cpu().numpy().view(np.uint16) == rres.view(np.uint16)).all()   # f16(a+b) is exact arithmetic
    assert H.rel_err(nrm.cpu().numpy(), rnrm) <= 2e-3


@pytest.mark.parametrize("N,K", [(100, 64), (1000, 1024), (4099, 4096), (77, 100)])
@pytest.mark.parametrize("B", [1, 4, 5])
def test_matvec_f16_lm_head(dev, N, K, B):
    from ironmill_b200 import ops
    w = H.make_weight(N, K, seed=9)
    x = H.make_x(B, K, seed=9)
    ref = orc.matvec_f16(w, x, threads=8)
    y = ops.matvec_f16(_cuda(w), _cuda(x)).cpu().numpy()
    assert H.rel_err(y, ref) <= 2e-3


def test_invalid_arguments_are_reported(dev):
    from ironmill_b200 import CudaSysError, ops
    qw = H.QWeight(8, 128)
    w = qw.gpu(dev)
    x = _cuda(H.make_x(65, 128))
    with pytest.raises(CudaSysError):
        ops.matvec_affine(w, x)
    with pytest.raises(CudaSysError):
        ops.AffineWeight(dev, qw.packed, qw.scales, qw.zps, 8, 128, 128, 3)


@pytest.mark.parametrize("I,K", [(64, 128), (3072, 1024), (1000, 4096)])
@pytest.mark.parametrize("B", [1, 3])
def test_fused_residual_norm_ffn(dev, I, K, B):
    """residual + RMSNorm + gate/up + SiLU in one launch against the two oracle steps."""
    from ironmill_b200 import ops
    g = H.QWeight(I, K, awq=True, seed=41, name="gate")
    u = H.QWeight(I, K, seed=41, name="up", awq_vec=g.awq)
    a, b = H.make_x(B, K, seed=6, name="a"), H.make_x(B, K, seed=6, name="b")
    gamma = (1.0 + 0.1 * H.rng_for("gamma2").standard_normal(K)).astype(np.float16)
    nrm, res = orc.fused_residual_rms_norm(a, b, gamma, 1e-5)
    ref = orc.ffn_gate_up_act(g.packed, g.scales_f16, g.zps_f16, u.packed, u.scales_f16, u.zps_f16, nrm, I, K, 128, 4, awq=g.awq, threads=8)
    out, gres, gnrm = ops.fused_residual_norm_ffn(g.gpu(dev), u.gpu(dev), _cuda(a), _cuda(b), _cuda(gamma), 1e-5)
    assert (gres.cpu().numpy().view(np.uint16) == res.view(np.uint16)).all()
    assert H.rel_err(gnrm.cpu().numpy(), nrm) <= 2e-3
    assert H.rel_err(out.cpu().numpy(), ref) <= 5e-3
