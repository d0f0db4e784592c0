"""GPU parity against the reference's OWN compiled CUDA op (unmodified sources built into baseline/_ref by
baseline/install_ref.sh), on identical seeded inputs: forward and all gradients.  Skipped when that build is
absent.  Bounds: fp64 allclose defaults; fp32 1e-4 of the result's scale; bf16 tensor-core mode 1e-2 / 2e-2."""
import numpy as np
import pytest
import torch

from tests import _reference
from tests._util import make_problem

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not _reference.available(), reason="baseline/_ref not built")]


@pytest.fixture(scope="module")
def ref():
    torch.backends.cuda.matmul.allow_tf32 = False
    mod = _reference.load("dconv_native")
    if mod is None:
        pytest.skip("reference extension does not import here")
    return mod


@pytest.fixture()
def ours():
    import d2conv3d_b200
    from d2conv3d_b200 import dconv_native
    d2conv3d_b200.set_math_mode("auto")
    yield dconv_native
    d2conv3d_b200.set_math_mode("auto")


def run(fn, p, dtype, mask=True, bias=True):
    ts = [torch.from_numpy(p[k]).cuda().requires_grad_() if p[k] is not None else None
          for k in ("x", "geo", "mask", "weight", "bias")]
    y = fn(*ts, p["stride"], p["padding"], p["dilation"], p["groups"], p["offset_groups"])
    y.backward(torch.from_numpy(p["gy"]).cuda())
    torch.cuda.synchronize()
    return [y.detach().cpu().numpy()] + [None if t is None else t.grad.cpu().numpy() for t in ts]


GEOMS = [
    dict(B=2, Cin=8, Cout=8, dims=(4, 9, 11), k=3, padding=1, G=2),
    dict(B=1, Cin=16, Cout=24, dims=(3, 8, 8), k=(1, 3, 3), padding=(0, 1, 1), stride=(1, 2, 2), G=4, groups=2),
    dict(B=3, Cin=6, Cout=6, dims=(5, 6, 7), k=(3, 1, 3), padding=(2, 0, 2), dilation=(2, 1, 2), G=3, groups=6),
    dict(B=1, Cin=64, Cout=64, dims=(4, 16, 16), k=3, padding=1, G=1),        # benchmark configuration 1
]
NAMES = ("y", "grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("gi", range(len(GEOMS)))
def test_generic_tier_matches_reference_cuda_op(ref, ours, gi, dtype):
    p = make_problem(700 + gi, dtype=dtype, offset_std=1.5, **GEOMS[gi])
    want = run(ref.deform_conv3d, p, dtype)
    got = run(ours.deform_conv3d, p, dtype)
    for nm, a, b in zip(NAMES, got, want):
        if dtype == np.float64:
            assert np.allclose(a, b, rtol=1e-5, atol=1e-8), (nm, np.abs(a - b).max())
        else:
            assert np.abs(a - b).max() <= 1e-4 * np.abs(b).max(), (nm, np.abs(a - b).max(), np.abs(b).max())


def test_no_mask_matches_reference(ref, ours):
    p = make_problem(710, 2, 4, 4, (3, 6, 6), padding=1, dtype=np.float64, mask=False, bias=False)
    want = run(ref.deform_conv3d, p, np.float64)
    got = run(ours.deform_conv3d, p, np.float64)
    for nm, a, b in zip(NAMES, got, want):
        if b is None:
            assert a is None
        else:
            assert np.allclose(a, b, rtol=1e-5, atol=1e-8), nm


def test_tensor_core_tier_matches_reference_cuda_op(ref, ours):
    import d2conv3d_b200
    p = make_problem(720, 2, 128, 128, (4, 12, 13), padding=1, G=2, dtype=np.float32, offset_std=2.0)
    want = run(ref.deform_conv3d, p, np.float32)
    d2conv3d_b200.set_math_mode("bf16")
    got = run(ours.deform_conv3d, p, np.float32)
    bounds = (1e-2, 2e-2, 2e-2, 2e-2, 2e-2, 2e-2)
    for nm, a, b, bound in zip(NAMES, got, want, bounds):
        assert np.abs(a - b).max() <= bound * np.abs(b).max(), (nm, np.abs(a - b).max() / np.abs(b).max())


def test_depthwise_matches_reference_cuda_op():
    refdw = _reference.load("fast_depthwise_conv3d")
    if refdw is None:
        pytest.skip("reference depthwise extension does not import here")
    from d2conv3d_b200 import fast_depthwise_conv3d as ours_dw
    torch.manual_seed(5)
    for stride, dilation, mult in ((1, 1, 1), (2, 1, 2), (1, 2, 1)):
        a = refdw.DepthwiseConv3d(6, 6 * mult, 3, stride=stride, padding=dilation, dilation=dilation).cuda()
        b = ours_dw.DepthwiseConv3d(6, 6 * mult, 3, stride=stride, padding=dilation, dilation=dilation).cuda()
        b.load_state_dict(a.state_dict())
        x1 = torch.randn(2, 6, 5, 9, 10, device="cuda", requires_grad=True)
        x2 = x1.detach().clone().requires_grad_()
        y1, y2 = a(x1), b(x2)
        gy = torch.randn_like(y1)
        y1.backward(gy); y2.backward(gy)
        assert torch.allclose(y1, y2, atol=1e-5)
        assert torch.allclose(x1.grad, x2.grad, atol=1e-5)
        assert torch.allclose(a.weight.grad, b.weight.grad, atol=1e-4)
        assert torch.allclose(a.bias.grad, b.bias.grad, atol=1e-4)
