"""GPU tests of deform_conv1d (evaluated by the 3-D kernels on a [B, C, 1, 1, L] view), following
ops/dconv-native/test/test_deform_conv.py:232-262: identity with conv1d for zero offsets, stride, groups,
float64 gradcheck; plus the numpy restatement of the reference's 1-D kernel as the oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dn():
    from d2conv3d_b200 import _lib, dconv_native
    _lib.lib()
    return dconv_native


def make(seed, B, C, Cout, L, K, stride=1, pad=0, dil=1, groups=1, G=1, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    Lo = (L + 2 * pad - dil * (K - 1) - 1) // stride + 1
    x = torch.randn(B, C, L, generator=g, dtype=dtype)
    off = torch.randn(B, G * K, Lo, generator=g, dtype=dtype) * 1.5
    alpha = torch.sigmoid(torch.randn(B, G * K, Lo, generator=g, dtype=dtype))
    w = torch.randn(Cout, C // groups, K, generator=g, dtype=dtype) / (C * K) ** 0.5
    b = torch.randn(Cout, generator=g, dtype=dtype)
    return x, off, alpha, w, b


@pytest.mark.parametrize("cfg", [
    dict(B=2, C=8, Cout=6, L=33, K=3),
    dict(B=1, C=12, Cout=6, L=40, K=5, stride=2, pad=2, dil=2, groups=3, G=2),
    dict(B=2, C=64, Cout=64, L=300, K=3, pad=1),          # a shape the tensor-core tier takes
])
def test_deform_conv1d_vs_oracle(dn, cfg):
    x, off, alpha, w, b = make(11, **cfg)
    kw = dict(stride=cfg.get("stride", 1), padding=cfg.get("pad", 0), dilation=cfg.get("dil", 1))
    y = dn.deform_conv1d(x.cuda(), off.cuda(), alpha.cuda(), w.cuda(), b.cuda(), n_weight_groups=cfg.get("groups", 1),
                         n_offset_groups=cfg.get("G", 1), **kw).cpu().numpy()
    want = orc.deform_conv1d_fwd(x.double().numpy(), off.double().numpy(), alpha.double().numpy(), w.double().numpy(),
                                 b.double().numpy(), groups=cfg.get("groups", 1), offset_groups=cfg.get("G", 1), **kw)
    assert y.shape == want.shape
    assert np.abs(y - want).max() <= 1e-4 * np.abs(want).max()


def test_no_deformation_is_conv1d(dn):
    x, off, alpha, w, b = make(12, B=2, C=24, Cout=6, L=256, K=3, groups=3)
    y = dn.deform_conv1d(x.cuda(), torch.zeros_like(off).cuda(), torch.ones_like(alpha).cuda(), w.cuda(), b.cuda(),
                         n_weight_groups=3)
    ref = torch.nn.functional.conv1d(x.cuda(), w.cuda(), b.cuda(), groups=3)
    assert torch.allclose(y, ref, atol=1e-5)


def test_gradcheck_float64(dn):
    x, off, alpha, w, b = make(13, B=1, C=4, Cout=2, L=9, K=3, pad=1, G=2, dtype=torch.float64)
    off = off + 0.25 * torch.sign(off)      # keep samples away from integer coordinates (kinks of the interpolation)
    args = [t.cuda().requires_grad_() for t in (x, off, alpha, w, b)]
    fn = lambda x_, o_, a_, w_, b_: dn.deform_conv1d(x_, o_, a_, w_, b_, padding=1, n_offset_groups=2)
    assert torch.autograd.gradcheck(fn, args, nondet_tol=1e-6)


def test_module_and_defaults(dn):
    m = dn.DeformConv1d(8, 4, 3, padding=1).cuda()
    x = torch.randn(2, 8, 20, device="cuda")
    off = torch.zeros(2, 3, 20, device="cuda")
    y = m(x, off, None)
    ref = torch.nn.functional.conv1d(x, m.weight, m.bias, padding=1)
    assert torch.allclose(y, ref, atol=1e-5)
