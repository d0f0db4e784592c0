"""GPU checks at the full sizes of the benchmark configurations, where the CPU oracle is too slow: properties
that do not depend on size (the identities the reference's own test-suite uses,
ops/dconv-native/test/test_deform_conv.py:262-330 and test_modules.py:48-67) checked against cuDNN / PyTorch,
and -- when baseline/_ref holds the reference's compiled op -- the reference's own CUDA kernels on the same
seeded inputs.  fp32-parity mode ("auto"): 1e-4 of the result's scale."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tests import _reference

pytestmark = pytest.mark.gpu

REL = 1e-4


@pytest.fixture()
def dn():
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    d2conv3d_b200.set_math_mode("auto")
    yield dconv_native
    d2conv3d_b200.set_math_mode("auto")
    _lib.device_status()


def rel(a, b):
    return float((a - b).abs().max() / b.abs().max())


def c2_inputs(seed=1002, B=2, C=512, dims=(8, 30, 54), G=8):
    g = torch.Generator().manual_seed(seed)
    V = dims
    x = torch.randn((B, C) + V, generator=g)
    off = torch.randn((B, G * 81) + V, generator=g) * 2.0
    mask = torch.sigmoid(torch.randn((B, G * 27) + V, generator=g))
    w = torch.randn((C, C, 3, 3, 3), generator=g) * (2.0 / (C * 27)) ** 0.5
    b = torch.randn(C, generator=g)
    gy = torch.randn((B, C) + V, generator=g)
    return [t.cuda() for t in (x, off, mask, w, b, gy)]


def test_c2_zero_offsets_unit_mask_is_conv3d(dn):
    x, off, mask, w, b, gy = c2_inputs()
    y = dn.deform_conv3d(x, torch.zeros_like(off), torch.ones_like(mask), w, b, 1, 1, 1, 1, 8)
    ref = F.conv3d(x.double(), w.double(), b.double(), padding=1).float()
    assert rel(y, ref) <= REL


def test_c2_integer_shift_is_conv3d_of_shifted_input(dn):
    """All offsets (+1, -1, +2) voxels == convolution of the input shifted by that amount with zero fill."""
    x, off, mask, w, b, gy = c2_inputs()
    o = torch.zeros_like(off)
    o[:, 0::3], o[:, 1::3], o[:, 2::3] = 1.0, -1.0, 2.0
    y = dn.deform_conv3d(x, o, None, w, None, 1, 1, 1, 1, 8)
    xs = torch.zeros_like(x)
    xs[:, :, :-1, 1:, :-2] = x[:, :, 1:, :-1, 2:]
    ref = F.conv3d(xs.double(), w.double(), None, padding=1).float()
    # at the border the deformable op also samples real voxels from padded base positions; compare the interior
    inner = (slice(None), slice(None), slice(1, -1), slice(1, -1), slice(1, -1))
    assert rel(y[inner], ref[inner]) <= REL


def test_c2_linearity_in_input_and_weight(dn):
    x, off, mask, w, b, gy = c2_inputs()
    x2 = torch.randn_like(x)
    f = lambda x_, w_: dn.deform_conv3d(x_, off, mask, w_, None, 1, 1, 1, 1, 8)
    y1, y2, y12 = f(x, w), f(x2, w), f(x + 2 * x2, w)
    assert rel(y12, y1 + 2 * y2) <= REL
    assert rel(f(x, -3 * w), -3 * y1) <= REL


@pytest.mark.skipif(not _reference.available(), reason="baseline/_ref not built")
def test_c2_full_size_matches_reference_cuda_op(dn):
    ref = _reference.load("dconv_native")
    if ref is None:
        pytest.skip("reference extension does not import here")
    x, off, mask, w, b, gy = c2_inputs()

    def run(fn, dtype=torch.float32):
        ts = [t.detach().to(dtype).requires_grad_() for t in (x, off, mask, w, b)]
        y = fn(*ts, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 8)
        y.backward(gy.to(dtype))
        torch.cuda.synchronize()
        return [y.detach()] + [t.grad for t in ts]

    want = run(ref.deform_conv3d)
    got = run(dn.deform_conv3d)
    names = ("y", "grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")
    for name, a, r in zip(names, got, want):
        assert rel(a, r) <= REL, (name, rel(a, r))
    # element-wise as well: |a - r| <= 1e-4 |r| + 1e-5 scale, so that small elements are held to a relative bound,
    # not only to the tensor's largest value.  The comparator for the results that are continuous in the sampling
    # position is the reference op in float64 (its fp32 run carries rounding noise of its own); grad_offset jumps
    # where a position crosses an integer, so it keeps the fp32 run, whose position arithmetic is this library's.
    want64 = run(ref.deform_conv3d, torch.float64)
    for name, a, r32, r64 in zip(names, got, want, want64):
        r = r32.double() if name == "grad_offset" else r64
        scale = float(r.abs().max())
        excess = float(((a.double() - r).abs() - 1e-4 * r.abs()).max()) / scale
        print(f"c2 auto {name}: max(|a-r| - 1e-4|r|)/scale = {excess:.2e}")
        assert excess <= 1e-5, (name, excess)


def test_c3_field_of_twos_is_dilated_conv3d(dn):
    """Size field == 2 everywhere <=> a dilation-2 convolution (network/layers.py semantics, test_modules.py:48-67)."""
    g = torch.Generator().manual_seed(1003)
    x = torch.randn((4, 256, 8, 60, 108), generator=g).cuda()
    w = (torch.randn((256, 256, 3, 3, 3), generator=g) * (2.0 / (256 * 27)) ** 0.5).cuda()
    field = torch.full((4, 3, 8, 60, 108), 2.0, device="cuda")
    y = dn.dyn_dilated_conv3d(x, field, None, w, None, "xyz", 1, 1, 1, 1, 1)
    # base grid -1,0,1 (dilation 1, padding 1) plus offsets base*(2-1): sampling at -2,0,2 around the voxel
    ref = F.conv3d(x, w, None, padding=2, dilation=2)
    assert rel(y, ref) <= REL


def test_c4_depthwise_full_size_matches_cudnn():
    from d2conv3d_b200 import fast_depthwise_conv3d
    torch.backends.cudnn.allow_tf32 = False
    g = torch.Generator().manual_seed(1004)
    x = torch.randn((8, 1024, 8, 30, 54), generator=g).cuda().requires_grad_()
    w = (torch.randn((1024, 1, 3, 3, 3), generator=g) * 0.1).cuda().requires_grad_()
    gy = torch.randn((8, 1024, 8, 30, 54), generator=g).cuda()
    y = fast_depthwise_conv3d._ops.depthwise_separable_conv3d(x, w, None, 1, 1, 1)
    y.backward(gy)
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    ref = F.conv3d(x, w, None, padding=1, groups=1024)
    ref.backward(gy)
    assert rel(y.detach(), ref.detach()) <= 1e-5
    assert rel(gx, x.grad) <= 1e-5
    assert rel(gw, w.grad) <= 1e-4      # 830 k-term sums, fp32 both sides
