"""CPU tests that pin the oracle (oracle/d2c_oracle.c) to the reference:
  * forward vs the reference's executable specification `expected_fn`
    (fixtures made by tests/golden/make_golden.py), float64 allclose defaults as in
    ops/dconv-native/test/test_deform_conv.py:204-214;
  * the conv3d identities of that suite (:347-371, :486-505);
  * offsets_from_size_map bit-exact vs the reference function's outputs;
  * backward vs central finite differences of the pinned forward (float64), which is
    what the reference's gradcheck-based backward tests establish;
  * the dynamic-dilated composition and the depthwise op vs PyTorch's CPU conv3d.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as orc
from tests import _util
from tests._util import deform_case_names, load_deform_case, make_problem, size_map_cases


@pytest.mark.parametrize("name", deform_case_names())
def test_forward_matches_reference_expected_fn_f64(name):
    c = load_deform_case(name, np.float64)
    y = orc.deform_conv3d_fwd(c["x"], c["offset"], c["mask"], c["weight"], c["bias"], c["stride"], c["padding"],
                              c["dilation"], c["groups"], c["offset_groups"])
    assert y.shape == c["expected"].shape
    assert np.allclose(y, c["expected"], rtol=1e-5, atol=1e-8), np.abs(y - c["expected"]).max()


@pytest.mark.parametrize("name", deform_case_names())
def test_forward_matches_reference_expected_fn_f32(name):
    c = load_deform_case(name, np.float32)
    y = orc.deform_conv3d_fwd(c["x"], c["offset"], c["mask"], c["weight"], c["bias"], c["stride"], c["padding"],
                              c["dilation"], c["groups"], c["offset_groups"])
    scale = np.abs(c["expected"]).max()
    # 1e-4 relative (to the output scale): the fp32 parity bound of the path
    assert np.abs(y - c["expected"]).max() <= 1e-4 * scale


@pytest.mark.parametrize("dtype,atol", [(np.float64, 1e-7), (np.float32, 1e-4)])
def test_no_deformation_equals_conv3d(dtype, atol):
    p = make_problem(1, 2, 3, 2, (5, 5, 5), dtype=dtype)
    off = np.zeros_like(p["geo"])
    ones = np.ones_like(p["mask"])
    y = orc.deform_conv3d_fwd(p["x"], off, ones, p["weight"], p["bias"])
    ref = F.conv3d(torch.from_numpy(p["x"]), torch.from_numpy(p["weight"]), torch.from_numpy(p["bias"])).numpy()
    assert np.allclose(y, ref, atol=atol)


def test_known_offset_equals_shifted_conv3d():
    p = make_problem(2, 2, 3, 2, (5, 5, 5), dtype=np.float64)
    off = np.ones_like(p["geo"])
    ones = np.ones_like(p["mask"])
    x = torch.from_numpy(p["x"])
    shifted = F.pad(x[:, :, 1:, 1:, 1:], (0, 1, 0, 1, 0, 1))
    ref = F.conv3d(shifted, torch.from_numpy(p["weight"]), torch.from_numpy(p["bias"])).numpy()
    y = orc.deform_conv3d_fwd(p["x"], off, ones, p["weight"], p["bias"])
    assert np.allclose(y, ref, atol=1e-7)


def test_groups_no_deformation_equals_grouped_conv3d():
    p = make_problem(3, 2, 12, 6, (4, 5, 6), padding=1, groups=3, G=2, dtype=np.float64)
    y = orc.deform_conv3d_fwd(p["x"], np.zeros_like(p["geo"]), np.ones_like(p["mask"]), p["weight"], p["bias"],
                              padding=1, groups=3, offset_groups=2)
    ref = F.conv3d(torch.from_numpy(p["x"]), torch.from_numpy(p["weight"]), torch.from_numpy(p["bias"]),
                   padding=1, groups=3).numpy()
    assert np.allclose(y, ref, atol=1e-7)


def test_offsets_from_size_map_bit_exact():
    s = size_map_cases()
    for n in s["names"]:
        kd = [int(v) for v in s[f"{n}/kd"]]
        mode = str(n).split("_")[0]
        o = orc.offsets_from_size_map(s[f"{n}/size_map"], mode, tuple(kd[:3]), tuple(kd[3:]))
        assert np.array_equal(o, s[f"{n}/offsets"]), n


def _numeric_grad(f, a, gy, eps=1e-6):
    """d(sum(f * gy))/da by central differences over every element of `a` (float64)."""
    g = np.zeros_like(a)
    flat, gflat = a.reshape(-1), g.reshape(-1)
    for i in range(flat.size):
        old = flat[i]
        flat[i] = old + eps
        fp = (f() * gy).sum()
        flat[i] = old - eps
        fm = (f() * gy).sum()
        flat[i] = old
        gflat[i] = (fp - fm) / (2 * eps)
    return g


@pytest.mark.parametrize("cfg", [
    dict(B=1, Cin=2, Cout=2, dims=(3, 3, 4), k=(2, 3, 2), padding=(1, 1, 0), G=1, groups=1),
    dict(B=2, Cin=4, Cout=4, dims=(2, 3, 3), k=(1, 3, 3), padding=(0, 1, 1), stride=(1, 2, 1), G=2, groups=2),
    dict(B=1, Cin=2, Cout=2, dims=(3, 4, 3), k=3, padding=1, dilation=(1, 2, 1), G=1, groups=1, mask=False),
])
def test_backward_matches_finite_differences(cfg):
    cfg = dict(cfg)
    use_mask = cfg.pop("mask", True)
    p = make_problem(11, dtype=np.float64, offset_std=0.7, mask=use_mask, **cfg)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=p["groups"],
              offset_groups=p["offset_groups"])
    # keep sampling positions away from integer coordinates, where the op is not differentiable
    frac = p["geo"] - np.floor(p["geo"])
    p["geo"] = np.where(frac < 0.05, p["geo"] + 0.1, np.where(frac > 0.95, p["geo"] - 0.1, p["geo"]))
    f = lambda: orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
    gx, goff, gmask, gw, gb = orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, **kw)
    assert np.allclose(gx, _numeric_grad(f, p["x"], p["gy"]), rtol=1e-5, atol=1e-6)
    assert np.allclose(goff, _numeric_grad(f, p["geo"], p["gy"]), rtol=1e-4, atol=1e-5)
    if use_mask:
        assert np.allclose(gmask, _numeric_grad(f, p["mask"], p["gy"]), rtol=1e-5, atol=1e-6)
    else:
        assert gmask is None
    assert np.allclose(gw, _numeric_grad(f, p["weight"], p["gy"]), rtol=1e-5, atol=1e-6)
    assert np.allclose(gb, _numeric_grad(f, p["bias"], p["gy"]), rtol=1e-5, atol=1e-6)


def test_gradient_at_border_coordinate_minus_one():
    """Zero offsets with pad 1: border taps sit at coordinate exactly -1, where the forward
    early-outs to 0 but the coordinate gradient is the right-sided difference
    (reference dconv3d_gpu.cu:59-61 vs :719-753)."""
    p = make_problem(5, 1, 1, 1, (3, 3, 3), padding=1, dtype=np.float64, bias=False)
    off = np.zeros_like(p["geo"])
    ones = np.ones_like(p["mask"])
    gy = np.zeros_like(p["gy"]); gy[0, 0, 0, 0, 0] = 1.0
    _, goff, _, _, _ = orc.deform_conv3d_bwd(gy, p["x"], off, ones, p["weight"], False, padding=1)
    # tap 0 = (-1,-1,-1) of voxel (0,0,0): z derivative = w[tap0] * (x[0,0,0]*(1-dx)(1-dy) - 0) with dx=dy=0 -> 0
    # because y0 = x0 = -1 are outside as well; tap 4 = (-1,0,0): z-derivative = w * (x[0,0,0] - 0)
    w = p["weight"].reshape(-1)
    V = 27
    assert goff[0, 3 * 4 + 0].reshape(-1)[0] == pytest.approx(w[4] * p["x"][0, 0, 0, 0, 0])
    assert goff[0, 3 * 0 + 0].reshape(-1)[0] == 0.0
    assert goff.reshape(1, 27, 3, V).shape == (1, 27, 3, V)


@pytest.mark.parametrize("mode", ["x", "xy", "xxz", "xyz"])
def test_dyn_dilated_equals_composition(mode):
    from d2conv3d_b200.dconv_native.grid import offsets_from_size_map
    G = 2
    p = make_problem(21, 2, 4, 4, (3, 5, 6), padding=1, G=G, dtype=np.float64, field_mode=mode)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=G)
    y = orc.dyn_dilated_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], mode, **kw)
    # reference composition in PyTorch autograd (utils/grid.py:72-98 + repeat per group)
    x, s, m, w, b = (torch.from_numpy(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias"))
    off = offsets_from_size_map(s, mode, (3, 3, 3), (1, 1, 1)).repeat(1, G, 1, 1, 1)
    y2 = orc.deform_conv3d_fwd(p["x"], off.detach().numpy(), p["mask"], p["weight"], p["bias"], **kw)
    assert np.array_equal(y, y2)
    gx, gs, gm, gw, gb = orc.dyn_dilated_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, mode, **kw)
    _, goff, _, _, _ = orc.deform_conv3d_bwd(p["gy"], p["x"], off.detach().numpy(), p["mask"], p["weight"], True, **kw)
    off.backward(torch.from_numpy(goff))
    assert np.allclose(gs, s.grad.numpy(), rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("stride,dilation,mult,bias", [(1, 1, 1, True), (2, 1, 2, False), (1, 2, 1, False), (2, 2, 2, True)])
@pytest.mark.parametrize("dtype,atol", [(np.float64, 1e-10), (np.float32, 1e-5)])
def test_depthwise_matches_torch_cpu(stride, dilation, mult, bias, dtype, atol):
    rng = np.random.default_rng(3)
    C, size = 2, 6
    pad = dilation
    x = (rng.standard_normal((2, C, size, size, size)) / 2).astype(dtype)
    w = rng.standard_normal((C * mult, 1, 3, 3, 3)).astype(dtype)
    b = rng.standard_normal((C * mult,)).astype(dtype) if bias else None
    xt, wt = torch.from_numpy(x).requires_grad_(), torch.from_numpy(w).requires_grad_()
    bt = torch.from_numpy(b).requires_grad_() if bias else None
    ref = F.conv3d(xt, wt, bt, stride=stride, padding=pad, dilation=dilation, groups=C)
    y = orc.depthwise_conv3d_fwd(x, w, b, stride, pad, dilation)
    assert np.allclose(y, ref.detach().numpy(), atol=atol)
    gy = (rng.standard_normal(ref.shape) / 2).astype(dtype)
    ref.backward(torch.from_numpy(gy))
    gx, gw, gb = orc.depthwise_conv3d_bwd(gy, x, w, bias, stride, pad, dilation)
    assert np.allclose(gx, xt.grad.numpy(), atol=atol)
    assert np.allclose(gw, wt.grad.numpy(), atol=atol * 10)
    if bias:
        assert np.allclose(gb, bt.grad.numpy(), atol=atol * 10)


def test_oracle_deform_conv1d_identities():
    """The 1-D oracle reduces to a plain (grouped, strided, dilated) convolution for zero offsets and unit
    modulation, and to a shifted one for integer offsets (ops/dconv-native/test/test_deform_conv.py:232-262)."""
    import torch
    rng = np.random.default_rng(21)
    B, C, Cout, L, K, groups = 2, 6, 4, 19, 3, 2
    x = rng.standard_normal((B, C, L)); w = rng.standard_normal((Cout, C // groups, K)); b = rng.standard_normal(Cout)
    for stride, pad, dil in ((1, 0, 1), (2, 2, 2)):
        Lo = (L + 2 * pad - dil * (K - 1) - 1) // stride + 1
        off = np.zeros((B, K, Lo))
        y = orc.deform_conv1d_fwd(x, off, None, w, b, stride, pad, dil, groups, 1)
        ref = torch.nn.functional.conv1d(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b), stride, pad,
                                         dil, groups).numpy()
        assert np.allclose(y, ref, atol=1e-12)
    # integer offset +1 on every tap == convolution of the input shifted left by one (zero fill)
    off = np.ones((B, K, L - K + 1))
    xs = np.concatenate([x[:, :, 1:], np.zeros((B, C, 1))], axis=2)
    y = orc.deform_conv1d_fwd(x, off, None, w, b, 1, 0, 1, groups, 1)
    ref = torch.nn.functional.conv1d(torch.from_numpy(xs), torch.from_numpy(w), torch.from_numpy(b), 1, 0, 1, groups).numpy()
    assert np.allclose(y, ref, atol=1e-12)


@pytest.mark.parametrize("name", _util.deform1d_case_names())
def test_deform_conv1d_matches_reference_expected_fn(name):
    """The 1-D oracle against outputs of the reference's own executable specification, expected_fn(1, ...)
    (ops/dconv-native/test/test_deform_conv.py:127-191), stored by tests/golden/make_golden.py."""
    c = _util.load_deform1d_case(name)
    y = orc.deform_conv1d_fwd(c["x"], c["offset"], c["mask"], c["weight"], c["bias"], c["stride"], c["padding"],
                              c["dilation"], c["groups"], c["offset_groups"])
    assert y.shape == c["expected"].shape
    assert np.allclose(y, c["expected"], rtol=1e-5, atol=1e-8)


def test_deform_conv1d_backward_matches_finite_differences():
    """Away from integer positions the 1-D op is differentiable: central differences of the pinned forward."""
    rng = np.random.default_rng(31)
    B, C, Cout, L, K, G, groups = 2, 4, 4, 11, 3, 2, 2
    stride, pad, dil = 2, 2, 1
    Lo = (L + 2 * pad - dil * (K - 1) - 1) // stride + 1
    x = rng.standard_normal((B, C, L)); w = rng.standard_normal((Cout, C // groups, K)); b = rng.standard_normal(Cout)
    off = rng.standard_normal((B, G * K, Lo)) * 1.5
    off = np.floor(off) + 0.2 + 0.6 * rng.random(off.shape)              # fractions in [0.2, 0.8]
    alpha = rng.random((B, G * K, Lo)) + 0.5
    gy = rng.standard_normal((B, Cout, Lo))
    kw = dict(stride=stride, padding=pad, dilation=dil, groups=groups, offset_groups=G)
    gx, goff, galpha, gw, gb = orc.deform_conv1d_bwd(gy, x, off, alpha, w, True, **kw)
    f = lambda x_, o_, a_, w_, b_: float((orc.deform_conv1d_fwd(x_, o_, a_, w_, b_, **kw) * gy).sum())
    eps = 1e-6
    for name, arr, grad, idx in (("x", x, gx, (1, 2, 5)), ("offset", off, goff, (0, 4, 3)), ("alpha", alpha, galpha, (1, 1, 2)),
                                 ("w", w, gw, (2, 1, 1)), ("b", b, gb, (3,))):
        args = dict(x=x, offset=off, alpha=alpha, w=w, b=b)
        hi, lo = arr.copy(), arr.copy()
        hi[idx] += eps; lo[idx] -= eps
        vals = []
        for v in (hi, lo):
            a2 = dict(args); a2[name] = v
            vals.append(f(a2["x"], a2["offset"], a2["alpha"], a2["w"], a2["b"]))
        fd = (vals[0] - vals[1]) / (2 * eps)
        assert abs(fd - grad[idx]) <= 1e-6 * max(1.0, abs(fd)), (name, fd, grad[idx])


def test_deform_conv1d_backward_integer_position_rule():
    """At an integer sampling position the reference's 1-D kernel moves the left neighbour one cell further left
    (dconv1d_gpu.cu:334-337): grad_offset = alpha * (x[p+1] - x[p-1]) * dcol and grad_alpha = x[p+1] * dcol."""
    x = np.array([[[1.0, 4.0, 9.0, 16.0, 25.0]]])          # B = C = 1, L = 5
    w = np.array([[[2.0]]])                                 # Cout = 1, K = 1
    off = np.zeros((1, 1, 5)); off[0, 0, 2] = 1.0           # position 2 samples cell 3 exactly
    alpha = np.full((1, 1, 5), 0.5)
    gy = np.ones((1, 1, 5))
    gx, goff, galpha, gw, gb = orc.deform_conv1d_bwd(gy, x, off, alpha, w, True)
    dcol = 2.0
    assert goff[0, 0, 2] == 0.5 * (25.0 - 9.0) * dcol       # cells 4 and 2 around the sampled cell 3
    assert galpha[0, 0, 2] == 25.0 * dcol                   # lerp(x[2], x[4], 1) = x[4]
    assert goff[0, 0, 0] == 0.5 * (4.0 - 0.0) * dcol        # position 0: left neighbour -1 is outside -> 0
    assert goff[0, 0, 4] == 0.5 * (0.0 - 16.0) * dcol       # position 4: right neighbour 5 is outside -> 0
    # the scatter keeps the ordinary corners: all of the gradient goes to the sampled cell
    assert gx[0, 0, 3] == 0.5 * dcol + 0.5 * dcol           # from positions 2 (offset +1) and 3
    assert gx[0, 0, 2] == 0.0


def test_oracle_thread_count_can_be_set_explicitly():
    """The timing legs of the bench set the OpenMP team size themselves (a launcher may export OMP_NUM_THREADS=1);
    results do not depend on it."""
    from tests._util import make_problem
    p = make_problem(77, 1, 4, 4, (2, 4, 4), padding=1, dtype=np.float64)
    before = orc.set_threads(0)
    try:
        assert orc.set_threads(2) == 2
        y2 = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], padding=1)
        assert orc.set_threads(1) == 1
        y1 = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], padding=1)
        assert np.array_equal(y1, y2)
    finally:
        orc.set_threads(before)
