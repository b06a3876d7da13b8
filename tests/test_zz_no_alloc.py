"""The attention entry point for hosts that cannot allocate device memory (an arena-owning server, a plugin
whose host forbids cudaMalloc after start-up): same inputs, same outputs as the ordinary entry point, with the
split partials in the library's built-in 4 MiB array.  Collected last on purpose: a failure here cannot hide the
result of any other test in a run that stops at the first failure.  Runs alone or after the rest of the suite."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _c(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_static_scratch_attention_matches_the_allocating_entry_point_twice():
    from ironmill_b200 import CudaSysError, ops
    dev = ops.Device(0)
    tqc = orc.TqConstants(128, 8, seed=7)
    tq = ops.TurboQuant(dev, 128, 8, tqc.signs, tqc.qjl, tqc.k_levels, tqc.k_bounds, tqc.v_levels, tqc.v_bounds)
    nh, nkv, max_seq = 32, 8, 640
    kc, vc = (torch.zeros((1, nkv, max_seq, 128), dtype=torch.uint8, device="cuda") for _ in range(2))
    ks, kr, vs = (torch.zeros((1, nkv, max_seq), dtype=torch.float32, device="cuda") for _ in range(3))
    # calls in a row: each finds its predecessor's partials in the array; the third asks for 8 splits of a 5-token
    # context, so most of its splits are empty and must overwrite what the 600-token call left there
    for ctx, seed, splits in ((600, 1, 0), (97, 2, 0), (600, 3, 8), (5, 4, 8)):
        k, v = H.make_x(ctx, nkv * 128, seed, "K"), H.make_x(ctx, nkv * 128, seed, "V")
        tq.encode(_c(k), True, kc, ks, kr, nkv, max_seq, 0)
        tq.encode(_c(v), False, vc, vs, torch.zeros_like(kr), nkv, max_seq, 0)
        q = _c(H.make_x(1, nh * 128, seed, "q"))
        ref = tq.attention(q, kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, ctx - 1, num_splits=splits)
        got = ops.tq_attention_static(tq, q, kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, ctx - 1, num_splits=splits)
        torch.cuda.synchronize()
        # tolerance of the attention tests (2e-3 of the largest reference magnitude)
        assert H.rel_err(got.cpu().numpy(), ref.cpu().numpy()) <= 2e-3
    # a request beyond the built-in array is refused with the sizes in the message
    qbig = torch.zeros((64, nh * 128), dtype=torch.float16, device="cuda")
    with pytest.raises(CudaSysError) as e:
        ops.tq_attention_static(tq, qbig, kc, vc, ks, vs, kr, 0.0884, nh, nkv, max_seq, 0, num_splits=64)
    assert "built-in scratch" in str(e.value)
    # a split count chosen by the library shrinks until the request fits instead of being refused
    q16 = _c(H.make_x(16, nh * 128, 9, "q16"))
    kc16, vc16 = (torch.zeros((16, nkv, max_seq, 128), dtype=torch.uint8, device="cuda") for _ in range(2))
    ks16, kr16, vs16 = (torch.ones((16, nkv, max_seq), dtype=torch.float32, device="cuda") for _ in range(3))
    ref = tq.attention(q16, kc16, vc16, ks16, vs16, kr16, 0.0884, nh, nkv, max_seq, 599, nseq=16)
    got = ops.tq_attention_static(tq, q16, kc16, vc16, ks16, vs16, kr16, 0.0884, nh, nkv, max_seq, 599, nseq=16)
    torch.cuda.synchronize()
    assert H.rel_err(got.cpu().numpy(), ref.cpu().numpy()) <= 2e-3
