"""The forward keeps its blended operand tiles for the weight gradient of the matching backward (d2c_sample_cache):
the backward then streams them instead of gathering and blending every sample again, as the reference does
(csrc/ops/dconv3d_gpu.cu:1037-1060 re-runs deformable_im2col).  These tests check, through the Python mirror and the
C ABI under it, that

* with the cache the weight gradient comes from the streaming kernel and equals the oracle's within the mode's bound,
* every result of the step equals the run without the cache (same kernels for everything but grad_weight),
* a call pair that cannot use the cache (math mode changed in between, cache switched off, CUDA-core tier) silently
  takes the ordinary route.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests._util import make_problem

pytestmark = pytest.mark.gpu

BOUND = {"auto": 1e-4, "bf16": 2e-2}


@pytest.fixture(autouse=True)
def _restore():
    import d2conv3d_b200
    from d2conv3d_b200 import _lib
    _lib.lib()
    yield
    d2conv3d_b200.set_math_mode("auto")
    d2conv3d_b200.set_keep_samples(True)
    _lib.device_status()


def cu(a, grad=False):
    if a is None:
        return None
    t = torch.from_numpy(a).cuda()
    return t.requires_grad_(True) if grad else t


def step(p, keep, mode):
    """Forward + backward through the autograd mirror; returns outputs, gradients and the library's phase names."""
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    d2conv3d_b200.set_math_mode(mode)
    d2conv3d_b200.set_keep_samples(keep)
    ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
    gy = cu(p["gy"])
    _lib.profile_read(); _lib.profile_enable(True)
    y = dconv_native.deform_conv3d(*ts, p["stride"], p["padding"], p["dilation"], 1, p["offset_groups"])
    y.backward(gy)
    _lib.profile_enable(False)
    phases = [n for n, _ in _lib.profile_read()]
    return y.detach().cpu().numpy(), [t.grad.cpu().numpy() for t in ts], phases


CASES = [
    dict(B=1, Cin=64, Cout=64, dims=(4, 8, 8), G=1),                  # one slice per tap: odd slice count (27)
    dict(B=2, Cin=128, Cout=128, dims=(3, 7, 9), G=2),                # ragged last tile of each clip
    dict(B=1, Cin=128, Cout=64, dims=(3, 6, 8), G=1),                 # 128 channels per group
    dict(B=1, Cin=64, Cout=512, dims=(2, 8, 9), G=1),                 # two 256-column chunks of grad_out
    dict(B=1, Cin=64, Cout=320, dims=(2, 8, 9), G=1),                 # 256 + 64 columns
    dict(B=1, Cin=128, Cout=128, dims=(3, 8, 8), G=4),                # 32 channels per group: slices span two groups
    dict(B=2, Cin=64, Cout=64, dims=(8, 30, 40), G=1),                # 150 tiles: several voxel ranges, ring wraps
    dict(B=1, Cin=64, Cout=64, dims=(5, 9, 9), G=1, stride=(1, 2, 2), dilation=(2, 1, 1), padding=(2, 1, 1)),
]


@pytest.mark.parametrize("mode", ["auto", "bf16"])
@pytest.mark.parametrize("ci", range(len(CASES)))
def test_weight_gradient_from_kept_samples(ci, mode):
    cfg = dict(CASES[ci])
    cfg.setdefault("k", 3)
    cfg.setdefault("padding", 1)
    p = make_problem(4100 + ci, dtype=np.float32, offset_std=2.0, **cfg)
    rng = np.random.default_rng(77 + ci)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=p["offset_groups"])
    want_y = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
    p["gy"] = rng.standard_normal(want_y.shape).astype(np.float32)
    want = orc.deform_conv3d_bwd(p["gy"].astype(np.float64), p["x"].astype(np.float64), p["geo"].astype(np.float64),
                                 p["mask"].astype(np.float64), p["weight"].astype(np.float64), **kw)
    y1, g1, ph1 = step(p, True, mode)
    y0, g0, ph0 = step(p, False, mode)
    assert "bwd_dw_sm100_saved" in ph1 and "bwd_dw_sm100" not in ph1, ph1
    assert "bwd_dw_sm100" in ph0 and "bwd_dw_sm100_saved" not in ph0, ph0
    # the forward and the data-side backward are the same kernels on the same inputs
    assert np.abs(y1 - y0).max() <= 1e-6 * np.abs(y0).max()      # partial tiles meet through atomics
    for i in (0, 1, 2, 4):
        scale = np.abs(g0[i]).max()
        assert np.abs(g1[i] - g0[i]).max() <= 1e-6 * scale, i     # atomics: order may differ in the last bits
    gw_want = want[3]
    scale = np.abs(gw_want).max()
    e1 = np.abs(g1[3] - gw_want).max() / scale
    e0 = np.abs(g0[3] - gw_want).max() / scale
    print(f"case {ci} {mode}: grad_weight err kept {e1:.2e}  re-gathered {e0:.2e}")
    assert e1 <= BOUND[mode]


def test_mode_change_between_forward_and_backward_falls_back():
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    p = make_problem(4200, dtype=np.float32, offset_std=2.0, B=1, Cin=64, Cout=64, dims=(4, 8, 8), G=1, k=3, padding=1)
    d2conv3d_b200.set_math_mode("bf16")
    ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
    y = dconv_native.deform_conv3d(*ts, p["stride"], p["padding"], p["dilation"], 1, 1)
    d2conv3d_b200.set_math_mode("auto")                     # the backward now runs the hi/lo kernels
    _lib.profile_read(); _lib.profile_enable(True)
    y.backward(torch.ones_like(y))
    _lib.profile_enable(False)
    phases = [n for n, _ in _lib.profile_read()]
    assert "bwd_dw_sm100" in phases and "bwd_dw_sm100_saved" not in phases, phases
    want = orc.deform_conv3d_bwd(np.ones(y.shape), p["x"].astype(np.float64), p["geo"].astype(np.float64),
                                 p["mask"].astype(np.float64), p["weight"].astype(np.float64), padding=p["padding"],
                                 stride=p["stride"], dilation=p["dilation"], groups=1, offset_groups=1)
    assert np.abs(ts[3].grad.cpu().numpy() - want[3]).max() <= 1e-4 * np.abs(want[3]).max()


def test_no_cache_without_gradients_or_on_the_cuda_core_tier():
    import ctypes
    import d2conv3d_b200
    from d2conv3d_b200 import _lib
    L = _lib.lib()
    x = torch.zeros(1, 64, 4, 8, 8, device="cuda")
    w = torch.zeros(64, 64, 3, 3, 3, device="cuda")
    desc = _lib.make_desc(x, w, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 1)
    # operand image (2 tiles x 2 blocks x 14 slice pairs x {hi, lo} x 2 slices x 8 KB) + staged fp32 input + positions
    assert L.d2c_sample_cache_bytes(ctypes.byref(desc)) == 2 * 2 * 14 * 4 * 8192 + 256 * 64 * 4 + 27 * 256 * 16
    assert _lib.SampleCache.for_forward(desc, x.device, differentiated=False) is None
    d2conv3d_b200.set_math_mode("fp32")
    assert L.d2c_sample_cache_bytes(ctypes.byref(desc)) == 0
    d2conv3d_b200.set_math_mode("auto")
    cap = L.d2c_get_max_intermediate_elements()
    L.d2c_set_max_intermediate_elements(1000)
    try:
        assert L.d2c_sample_cache_bytes(ctypes.byref(desc)) == 0
    finally:
        L.d2c_set_max_intermediate_elements(cap)


@pytest.mark.parametrize("mode", ["auto", "bf16"])
def test_dilation_field_layer_with_fused_head_uses_kept_samples(mode):
    """The size-conditioned layer (predictor head fused) trains with the cache as well: gradients equal the run
    without it."""
    import d2conv3d_b200
    from d2conv3d_b200 import _lib
    from d2conv3d_b200.dconv_native import modules
    torch.manual_seed(5)
    d2conv3d_b200.set_math_mode(mode)
    layer = modules.XYZSizeConditionedMDConv3d(128, 64, 3, padding=1, offset_groups=2).cuda()
    with torch.no_grad():
        for q in layer.deform_params.parameters():
            q.normal_(0, 0.05)
    x = torch.randn(2, 128, 4, 10, 12, device="cuda")
    res = []
    for keep in (True, False):
        d2conv3d_b200.set_keep_samples(keep)
        layer.zero_grad()
        xi = x.clone().requires_grad_(True)
        _lib.profile_read(); _lib.profile_enable(True)
        y = layer(xi)
        y.square().mean().backward()
        _lib.profile_enable(False)
        phases = [n for n, _ in _lib.profile_read()]
        assert ("bwd_dw_sm100_saved" in phases) == keep, phases
        res.append([y.detach().clone(), xi.grad.clone()] + [q.grad.clone() for q in layer.parameters()])
    # both routes are within the mode's bound of the exact result; they differ in products formed and summation order
    tol = 1e-4 if mode == "auto" else 5e-3
    for a, b in zip(*res):
        assert (a - b).abs().max().item() <= tol * max(b.abs().max().item(), 1e-30)


def test_inference_under_no_grad_keeps_nothing(monkeypatch):
    """A forward under torch.no_grad() over a layer whose weights are trainable (the usual evaluation pass) must not
    keep samples: ctx.needs_input_grad is True there, so the decision is taken where the op is called."""
    from d2conv3d_b200 import _lib
    from d2conv3d_b200.dconv_native import modules
    seen = []
    real = _lib.SampleCache.for_forward

    def spy(desc, device, differentiated):
        seen.append(bool(differentiated))
        return real(desc, device, differentiated)

    monkeypatch.setattr(_lib.SampleCache, "for_forward", staticmethod(spy))
    layer = modules.XYZSizeConditionedMDConv3d(64, 64, 3, padding=1, offset_groups=1).cuda()
    x = torch.randn(1, 64, 4, 8, 8, device="cuda")
    with torch.no_grad():
        layer(x)
    assert seen == [False]
    layer(x)                       # weights require grad, grad mode on: a training forward
    assert seen == [False, True]
    layer.requires_grad_(False)
    layer(x)                       # nothing to differentiate
    assert seen == [False, True, False]
