"""GPU tests of deform_conv1d, following ops/dconv-native/test/test_deform_conv.py:232-340: the golden outputs of
the reference's expected_fn(1, ...), identity with conv1d for zero offsets, stride, groups, float64 gradcheck;
forward and all five gradients against the numpy restatement of the reference's 1-D kernels -- at fractional
AND at exactly-integer sampling positions, where the 1-D reference has a rule of its own (dconv1d_gpu.cu:334-337)
-- and against the reference's own compiled CUDA op when baseline/_ref is present."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import _reference, _util

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


@pytest.mark.parametrize("name", _util.deform1d_case_names())
def test_forward_matches_reference_expected_fn(dn, name):
    c = _util.load_deform1d_case(name)
    cu = lambda a: None if a is None else torch.from_numpy(a).cuda()
    y = dn.deform_conv1d(cu(c["x"]), cu(c["offset"]), cu(c["mask"]), cu(c["weight"]), cu(c["bias"]), c["stride"],
                         c["padding"], c["dilation"], c["groups"], c["offset_groups"]).cpu().numpy()
    assert np.allclose(y, c["expected"], rtol=1e-5, atol=1e-8)      # float64, the suite's allclose defaults


def _integerise(off, frac):
    """Every `frac`-th offset becomes an exact integer (the zero-initialised predictor's case)."""
    off = off.clone()
    flat = off.view(-1)
    flat[::frac] = torch.round(flat[::frac])
    return off


GRAD_CASES = [
    dict(B=2, C=8, Cout=6, L=33, K=3),
    dict(B=1, C=12, Cout=6, L=40, K=5, stride=2, pad=2, dil=2, groups=3, G=2),
    dict(B=2, C=64, Cout=64, L=150, K=3, pad=1),
]


@pytest.mark.parametrize("ci", range(len(GRAD_CASES)))
@pytest.mark.parametrize("integer_every", [0, 1, 3])
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_all_gradients_vs_oracle_including_integer_positions(dn, ci, integer_every, dtype):
    cfg = GRAD_CASES[ci]
    x, off, alpha, w, b = make(40 + ci, dtype=torch.float64, **cfg)
    if integer_every:
        off = _integerise(off, integer_every)
    Lo = off.shape[2]
    gy = torch.randn(x.shape[0], w.shape[0], Lo, generator=torch.Generator().manual_seed(50 + ci), dtype=torch.float64)
    kw = dict(stride=cfg.get("stride", 1), padding=cfg.get("pad", 0), dilation=cfg.get("dil", 1))
    g, G = cfg.get("groups", 1), cfg.get("G", 1)
    want_y = orc.deform_conv1d_fwd(x.numpy(), off.numpy(), alpha.numpy(), w.numpy(), b.numpy(), groups=g,
                                   offset_groups=G, **kw)
    want = orc.deform_conv1d_bwd(gy.numpy(), x.numpy(), off.numpy(), alpha.numpy(), w.numpy(), True, groups=g,
                                 offset_groups=G, **kw)
    ts = [t.to(dtype).cuda().requires_grad_() for t in (x, off, alpha, w, b)]
    y = dn.deform_conv1d(*ts, n_weight_groups=g, n_offset_groups=G, **kw)
    y.backward(gy.to(dtype).cuda())
    tol = 1e-10 if dtype == torch.float64 else 1e-4
    rel = lambda got, ref: float(np.abs(got.detach().cpu().double().numpy() - ref).max() / max(np.abs(ref).max(), 1e-30))
    assert rel(y, want_y) <= tol
    for name, t, ref in zip(("x", "offset", "alpha", "weight", "bias"), ts, want):
        assert rel(t.grad, ref) <= tol, (name, rel(t.grad, ref))


@pytest.mark.skipif(not _reference.available(), reason="baseline/_ref (the reference's compiled extension) is absent")
@pytest.mark.parametrize("ci", range(len(GRAD_CASES)))
@pytest.mark.parametrize("integer_every", [0, 1, 3])
def test_forward_and_all_gradients_vs_reference_cuda_op(dn, ci, integer_every):
    """Same seeded inputs through the reference's own deform_conv1d (unmodified sources) and through this library."""
    ref = _reference.load("dconv_native")
    if ref is None:
        pytest.skip("the reference extension did not import")
    cfg = GRAD_CASES[ci]
    x, off, alpha, w, b = make(60 + ci, dtype=torch.float64, **cfg)
    if integer_every:
        off = _integerise(off, integer_every)
    gy = torch.randn(x.shape[0], w.shape[0], off.shape[2], generator=torch.Generator().manual_seed(70 + ci),
                     dtype=torch.float64).cuda()
    kw = dict(stride=cfg.get("stride", 1), padding=cfg.get("pad", 0), dilation=cfg.get("dil", 1),
              n_weight_groups=cfg.get("groups", 1), n_offset_groups=cfg.get("G", 1))
    outs = []
    for fn in (ref.deform_conv1d, dn.deform_conv1d):
        ts = [t.cuda().requires_grad_() for t in (x, off, alpha, w, b)]
        y = fn(*ts, **kw)
        y.backward(gy)
        torch.cuda.synchronize()
        outs.append([y.detach()] + [t.grad for t in ts])
    for name, a, c in zip(("y", "grad_x", "grad_offset", "grad_alpha", "grad_weight", "grad_bias"), *outs):
        scale = max(float(a.abs().max()), 1e-30)
        assert float((a - c).abs().max()) <= 1e-10 * scale, name
