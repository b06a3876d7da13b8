"""GPU quantize-pack against the CPU oracle: bit-exact codes, scales and zero points."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _run(w, gs, bits, awq=None):
    from ironmill_b200 import ops
    wd = torch.from_numpy(w).cuda()
    ad = torch.from_numpy(awq).cuda() if awq is not None else None
    packed, scales, zps = ops.quantize_affine(wd, gs, bits, ad)
    torch.cuda.synchronize()
    return packed.cpu().numpy(), scales.cpu().numpy(), zps.cpu().numpy()


def _check(w, gs, bits, awq=None):
    codes, scales, zps = orc.quantize_groups(w, gs, bits, awq=awq, threads=8)
    ref_packed = orc.pack_int4(codes) if bits == 4 else codes.reshape(-1)
    packed, s, z = _run(w, gs, bits, awq)
    assert (s.view(np.uint32) == scales.view(np.uint32)).all(), "scales differ"
    assert (z.view(np.uint32) == zps.view(np.uint32)).all(), "zero points differ"
    assert (packed == ref_packed).all(), "codes differ"


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("awq", [False, True])
def test_config1_shape(bits, awq):
    # W [4096,4096] ~ N(0, 0.02), group 128
    w = H.make_weight(4096, 4096, seed=1)
    _check(w, 128, bits, H.make_awq(4096, 1) if awq else None)


@pytest.mark.parametrize("shape,gs", [((3, 6), 4), ((5, 7), 4), ((1, 1), 128), ((2, 130), 128), ((7, 96), 32), ((4, 256), 256)])
@pytest.mark.parametrize("bits", [4, 8])
def test_ragged_and_small(shape, gs, bits):
    # partial last group, odd K (4-bit pairs straddle rows), group larger than the row
    w = H.make_weight(*shape, seed=2, std=1.0)
    _check(w, gs, bits)


def test_known_answer_on_gpu():
    # affine_quantize.rs:585-598 replayed through the CUDA path
    w = np.array([[-3, 0, 3, 6, 12]], dtype=np.float16)
    packed, s, z = _run(w, 5, 4)
    assert s[0, 0] == 1.0 and z[0, 0] == 3.0
    assert orc.unpack_int4(packed, 5).tolist() == [0, 3, 6, 9, 15]


def test_degenerate_groups():
    w = np.zeros((4, 256), dtype=np.float16)
    w[1] = 42.0                       # uniform group: scale 1, zp = round(-min)
    w[2, :128] = np.float16(-0.0)     # signed zeros
    w[2, 5] = 0.0
    w[3, 3] = np.inf                  # non-finite values are skipped for min/max
    w[3, 4] = np.nan
    w[3, 130:] = np.nan
    w[3, 128:130] = np.inf
    _check(w, 128, 4)
    _check(w, 128, 8)


def test_empty_input():
    from ironmill_b200 import ops
    w = torch.empty((0, 128), dtype=torch.float16, device="cuda")
    packed, s, z = ops.quantize_affine(w, 128, 4)
    assert packed.numel() == 0 and s.numel() == 0


def test_full_size_property_dequant_error_bound():
    """Full gate+up size (28672 x 4096): every dequantised value lies within scale/2 of the
    input (size-independent round-trip property; the oracle is not run at this size)."""
    from ironmill_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    w = (torch.randn((28672, 4096), generator=g, device="cuda") * 0.02).half()
    packed, s, z = ops.quantize_affine(w, 128, 4)
    lo = (packed & 0xF).float()
    hi = (packed >> 4).float()
    q = torch.stack([lo, hi], dim=-1).reshape(28672, 32, 128)
    deq = (q - z[..., None]) * s[..., None]
    err = (deq - w.float().reshape(28672, 32, 128)).abs()
    assert bool((err <= s[..., None] * 0.5001 + 1e-7).all())
    assert int(q.max()) <= 15 and int(q.min()) >= 0
