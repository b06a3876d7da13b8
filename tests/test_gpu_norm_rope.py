"""Norm / embedding / RoPE kernels against the CPU oracle (fp16 outputs; tolerance 2e-3 of the
largest reference magnitude, residual sums bit-exact)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 2e-3


def _c(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _gamma(n, seed=0):
    return (1.0 + 0.1 * H.rng_for("gamma", seed).standard_normal(n)).astype(np.float16)


@pytest.mark.parametrize("Hd,T", [(64, 1), (1024, 3), (4096, 2), (100, 5)])
def test_rms_norm_and_residual(Hd, T):
    from ironmill_b200 import ops
    x, b, g = H.make_x(T, Hd, 1), H.make_x(T, Hd, 2, "b"), _gamma(Hd)
    assert H.rel_err(ops.rms_norm(_c(x), _c(g), 1e-6).cpu().numpy(), orc.rms_norm(x, g, 1e-6)) <= TOL
    n, r = ops.fused_residual_rms_norm(_c(x), _c(b), _c(g), 1e-5)
    rn, rr = orc.fused_residual_rms_norm(x, b, g, 1e-5)
    assert (r.cpu().numpy().view(np.uint16) == rr.view(np.uint16)).all()
    assert H.rel_err(n.cpu().numpy(), rn) <= TOL
    assert (ops.residual_add(_c(x), _c(b)).cpu().numpy().view(np.uint16) == orc.residual_add(x, b).view(np.uint16)).all()


def test_embedding_norm_with_out_of_range_token():
    from ironmill_b200 import ops
    vocab, Hd = 300, 1024
    table = H.make_weight(vocab, Hd, seed=3)
    g = _gamma(Hd, 1)
    tokens = np.array([0, 299, 300, 17, 4000000000], dtype=np.uint32)   # 300 and 4e9 are out of range -> zeros
    n, raw = ops.embedding_norm(_c(tokens.view(np.int32)), _c(table), _c(g), 1e-6, 1.0)
    rn, rraw = orc.embedding_norm(tokens, table, g, 1e-6, 1.0)
    assert (raw.cpu().numpy().view(np.uint16) == rraw.view(np.uint16)).all()
    assert H.rel_err(n.cpu().numpy(), rn) <= TOL
    assert not raw[2].any() and not raw[4].any() and not n[2].any()


def test_rope_table_matches_host_f64():
    from ironmill_b200 import ops
    for hd, theta, rd in ((128, 1e6, None), (128, 5e5, None), (64, 1e4, 32)):
        cos, sin = ops.rope_table(hd, 257, theta, rd)
        rc, rs = orc.rope_table(hd, 257, theta, rd)
        assert (cos.cpu().numpy().view(np.uint16) == rc.view(np.uint16)).all()
        assert (sin.cpu().numpy().view(np.uint16) == rs.view(np.uint16)).all()


@pytest.mark.parametrize("nh,nkv,hd,T,off,rd", [(16, 8, 128, 1, 0, None), (16, 8, 128, 3, 40, None), (4, 2, 64, 2, 7, 32), (32, 8, 128, 1, 511, None)])
def test_qk_norm_rope(nh, nkv, hd, T, off, rd):
    from ironmill_b200 import ops
    q, k = H.make_x(T, nh * hd, 4, "q"), H.make_x(T, nkv * hd, 4, "k")
    qw, kw = _gamma(hd, 2), _gamma(hd, 3)
    cos, sin = orc.rope_table(hd, 600, 1e6, rd)
    rq, rk = orc.qk_norm_rope(q, k, qw, kw, cos, sin, nh, nkv, hd, off, 1e-6, rd)
    qd, kd = _c(q), _c(k)
    ops.qk_norm_rope_(qd, kd, _c(qw), _c(kw), _c(cos), _c(sin), nh, nkv, hd, off, 1e-6, rd)
    assert H.rel_err(qd.cpu().numpy(), rq) <= TOL and H.rel_err(kd.cpu().numpy(), rk) <= TOL


def test_plain_rope_llama():
    from ironmill_b200 import ops
    heads, hd, T, off = 32, 128, 2, 100
    x = H.make_x(T, heads * hd, 6)
    cos, sin = orc.rope_table(hd, 256, 5e5)
    ref = orc.rope(x, cos, sin, heads, hd, off)
    xd = _c(x)
    ops.rope_(xd, _c(cos), _c(sin), heads, hd, off)
    assert H.rel_err(xd.cpu().numpy(), ref) <= 1e-3
