"""GPU parity tests of the deformable / dynamic-dilated conv3d path.  Every call goes
Python mirror -> ctypes -> C ABI of libd2conv3d.so -> CUDA kernels; results are compared
with the CPU oracle on identical seeded inputs and with the committed golden fixtures.

Bounds: integer corner indices bit-exact; float64 to allclose defaults (as the
reference's own suite); float32 within 1e-4 of the result's scale.
"""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from oracle import oracle as orc
from tests._util import deform_case_names, load_deform_case, make_problem

pytestmark = pytest.mark.gpu

REL_F32 = 1e-4


@pytest.fixture(scope="module")
def dn():
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    _lib.lib()                       # raises if the CUDA library is missing: no fallback
    assert torch.cuda.is_available()
    d2conv3d_b200.set_math_mode("auto")
    return dconv_native


def cu(a, grad=False):
    if a is None:
        return None
    t = torch.from_numpy(a).cuda()
    return t.requires_grad_() if grad else t


def close(got, want, dtype, what="", rel32=REL_F32):
    got = got.detach().cpu().numpy() if torch.is_tensor(got) else got
    assert got.shape == want.shape, what
    if dtype == np.float64:
        assert np.allclose(got, want, rtol=1e-5, atol=1e-8), f"{what}: max diff {np.abs(got - want).max()}"
    else:
        scale = max(np.abs(want).max(), 1e-30)
        err = np.abs(got - want).max()
        assert err <= rel32 * scale, f"{what}: max diff {err} vs scale {scale}"


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("name", deform_case_names())
def test_forward_golden(dn, name, dtype):
    c = load_deform_case(name, dtype)
    y = dn.deform_conv3d(cu(c["x"]), cu(c["offset"]), cu(c["mask"]), cu(c["weight"]), cu(c["bias"]), c["stride"],
                         c["padding"], c["dilation"], c["groups"], c["offset_groups"])
    close(y, c["expected"].astype(dtype), dtype, name)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("name", deform_case_names())
def test_backward_vs_oracle_on_golden_inputs(dn, name, dtype):
    c = load_deform_case(name, dtype)
    kw = dict(stride=c["stride"], padding=c["padding"], dilation=c["dilation"], groups=c["groups"],
              offset_groups=c["offset_groups"])
    rng = np.random.default_rng(7)
    gy = rng.standard_normal(c["expected"].shape).astype(dtype)
    want = orc.deform_conv3d_bwd(gy, c["x"], c["offset"], c["mask"], c["weight"], c["bias"] is not None, **kw)
    ts = [cu(c[k], True) for k in ("x", "offset", "mask", "weight", "bias")]
    y = dn.deform_conv3d(*ts, c["stride"], c["padding"], c["dilation"], c["groups"], c["offset_groups"])
    y.backward(cu(gy))
    for t, w_, nm in zip(ts, want, ("grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")):
        if t is None:
            assert w_ is None
            continue
        close(t.grad, w_, dtype, f"{name}/{nm}")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_integer_corners_bit_exact(dn, dtype):
    for name in ("pad1_big_offsets", "pad1_integer_offsets", "forward_mixed", "backward_geom"):
        c = load_deform_case(name, dtype)
        got = dn._ops.corners(c["x"].shape, c["weight"].shape[:1] + (c["x"].shape[1],) + c["weight"].shape[2:],
                              cu(c["offset"]), c["stride"], c["padding"], c["dilation"], c["offset_groups"])
        want = orc.deform_conv3d_corners(c["x"].shape, c["weight"].shape, c["offset"], c["stride"], c["padding"],
                                         c["dilation"], c["offset_groups"])
        assert np.array_equal(got.cpu().numpy(), want), name
    # offsets that land exactly on integers and on x.5 after the single fp add
    p = make_problem(3, 2, 4, 4, (4, 9, 11), padding=1, G=2, dtype=dtype)
    p["geo"] = np.round(p["geo"] * 2) / 2
    got = dn._ops.corners(p["x"].shape, p["weight"].shape, cu(p["geo"]), p["stride"], p["padding"], p["dilation"], 2)
    want = orc.deform_conv3d_corners(p["x"].shape, p["weight"].shape, p["geo"], p["stride"], p["padding"], p["dilation"], 2)
    assert np.array_equal(got.cpu().numpy(), want)


GEOMS = [
    dict(B=2, Cin=8, Cout=8, dims=(4, 9, 11), k=3, padding=1, G=2),
    dict(B=1, Cin=16, Cout=24, dims=(3, 8, 8), k=(1, 3, 3), padding=(0, 1, 1), stride=(1, 2, 2), G=4, groups=2),
    dict(B=3, Cin=6, Cout=6, dims=(5, 6, 7), k=(3, 1, 3), padding=(2, 0, 2), dilation=(2, 1, 2), G=3, groups=6),
    dict(B=2, Cin=70, Cout=66, dims=(3, 5, 13), k=3, padding=1, G=1),          # ragged tiles
]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("mask,bias", [(True, True), (False, False)])
@pytest.mark.parametrize("gi", range(len(GEOMS)))
def test_forward_backward_vs_oracle(dn, gi, mask, bias, dtype):
    p = make_problem(100 + gi, dtype=dtype, offset_std=1.5, mask=mask, bias=bias, **GEOMS[gi])
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=p["groups"],
              offset_groups=p["offset_groups"])
    want_y = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
    want_g = orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], bias, **kw)
    ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
    y = dn.deform_conv3d(*ts, p["stride"], p["padding"], p["dilation"], p["groups"], p["offset_groups"])
    close(y, want_y, dtype, "y")
    y.backward(cu(p["gy"]))
    for t, w_, nm in zip(ts, want_g, ("grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")):
        if t is not None:
            close(t.grad, w_, dtype, nm)


def test_baseline_config1_fp32(dn):
    """B=1, 64->64, 4x16x16, 3x3x3, pad 1, one offset group; offsets ~ N(0,1), mask = sigmoid(N(0,1)),
    Kaiming-normal weight, zero bias; forward and all five gradients."""
    p = make_problem(1001, 1, 64, 64, (4, 16, 16), padding=1, dtype=np.float32)
    p["bias"] = np.zeros_like(p["bias"])
    kw = dict(stride=1, padding=1, dilation=1, groups=1, offset_groups=1)
    want_y = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
    want_g = orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, **kw)
    ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
    y = dn.deform_conv3d(*ts, 1, 1, 1, 1, 1)
    close(y, want_y, np.float32, "y")
    y.backward(cu(p["gy"]))
    for t, w_, nm in zip(ts, want_g, ("grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")):
        close(t.grad, w_, np.float32, nm)


def test_reference_identities(dn):
    """test_no_deformation / test_known_offset of the reference suite
    (ops/dconv-native/test/test_deform_conv.py:347-371, :486-505)."""
    torch.manual_seed(0)
    x = torch.randn(2, 3, 5, 5, 5, dtype=torch.float64, device="cuda")
    w = torch.randn(2, 3, 3, 3, 3, dtype=torch.float64, device="cuda")
    b = torch.randn(2, dtype=torch.float64, device="cuda")
    off = torch.zeros(2, 81, 3, 3, 3, dtype=torch.float64, device="cuda")
    ones = torch.ones(2, 27, 3, 3, 3, dtype=torch.float64, device="cuda")
    assert torch.allclose(dn.deform_conv3d(x, off, ones, w, b), F.conv3d(x, w, b), atol=1e-7)
    shifted = F.pad(x[:, :, 1:, 1:, 1:], (0, 1, 0, 1, 0, 1))
    got = dn.deform_conv3d(x, torch.ones_like(off), ones, w, b)
    assert torch.allclose(got, F.conv3d(shifted, w, b), atol=1e-7)


@pytest.mark.parametrize("cfg", [
    dict(),
    dict(stride=3),
    dict(channels_in=6, channels_out=4, G=2),
    dict(channels_in=12, channels_out=6, groups=3),
    dict(channels_in=6, channels_out=6, groups=6, G=3),
    dict(dims=(2, 3, 5), k=(3, 5, 3), stride=(1, 2, 1), padding=(1, 3, 5), dilation=(1, 1, 2), channels_out=5),
    dict(no_mask=True),
    dict(no_bias=True),
])
def test_gradcheck_float64(dn, cfg):
    """The reference's backward tests: torch.autograd.gradcheck on all inputs, nondet_tol=1e-6."""
    cfg = dict(cfg)
    p = make_problem(55, 2, cfg.get("channels_in", 3), cfg.get("channels_out", 2), cfg.get("dims", (4, 4, 4)),
                     k=cfg.get("k", 3), stride=cfg.get("stride", 1), padding=cfg.get("padding", 0),
                     dilation=cfg.get("dilation", 1), groups=cfg.get("groups", 1), G=cfg.get("G", 1),
                     dtype=np.float64, mask=not cfg.get("no_mask"), bias=not cfg.get("no_bias"))
    ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
    fn = lambda x, o, m, w, b: dn.deform_conv3d(x, o, m, w, b, p["stride"], p["padding"], p["dilation"],
                                                 p["groups"], p["offset_groups"])
    assert torch.autograd.gradcheck(fn, ts, nondet_tol=1e-6)


def test_half_inputs_are_upcast(dn):
    x = torch.randn(2, 3, 5, 5, 5, device="cuda")
    off = torch.randn(2, 81, 3, 3, 3, device="cuda").half()
    m = torch.rand(2, 27, 3, 3, 3, device="cuda").half()
    w = torch.randn(2, 3, 3, 3, 3, device="cuda").half()
    assert dn.deform_conv3d(x, off, m, w).dtype == torch.float32


def test_shape_errors_raise_runtime_error(dn):
    x = torch.randn(2, 4, 5, 5, 5, device="cuda")
    w = torch.randn(4, 4, 3, 3, 3, device="cuda")
    with pytest.raises(RuntimeError):
        dn.deform_conv3d(x, torch.zeros(2, 80, 3, 3, 3, device="cuda"), None, w)
    with pytest.raises(RuntimeError):
        dn.deform_conv3d(x, torch.zeros(2, 81, 3, 3, 4, device="cuda"), None, w)
    with pytest.raises(RuntimeError):
        dn.deform_conv3d(x, torch.zeros(2, 81, 3, 3, 3, device="cuda"), torch.zeros(2, 26, 3, 3, 3, device="cuda"), w)
    with pytest.raises(RuntimeError):
        dn.deform_conv3d(x, torch.zeros(2, 81, 3, 3, 3, device="cuda"), None, w, n_offset_groups=3)


def test_intermediate_cap_slices_backward(dn):
    p = make_problem(77, 5, 4, 4, (3, 5, 5), padding=1, dtype=np.float32)
    def run():
        ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
        dn.deform_conv3d(*ts, 1, 1, 1, 1, 1).backward(cu(p["gy"]))
        return [t.grad.clone() for t in ts]
    full = run()
    old = dn._ops.config.get_max_intermediate_elements()
    try:
        dn._ops.config.set_max_intermediate_elements(2 * 4 * 27 * 75)   # two clips per slice
        sliced = run()
    finally:
        dn._ops.config.set_max_intermediate_elements(old)
    for a, b in zip(full, sliced):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)


# ---- dynamic-dilated conv ------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("mode", ["x", "xy", "xxz", "xyz"])
def test_dyn_dilated_vs_oracle(dn, mode, dtype):
    G = 2
    p = make_problem(200, 2, 8, 8, (4, 7, 9), padding=1, G=G, dtype=dtype, field_mode=mode)
    p["geo"][0, :, 0, 0, :] = 1.0      # field exactly 1 -> offset exactly 0 -> integer coordinates
    kw = dict(stride=1, padding=1, dilation=1, groups=1, offset_groups=G)
    got_c = dn._ops.field_corners(p["x"].shape, p["weight"].shape, cu(p["geo"]), mode, (1, 1, 1), (1, 1, 1), (1, 1, 1), G)
    want_c = orc.dyn_dilated_conv3d_corners(p["x"].shape, p["weight"].shape, p["geo"], mode, 1, 1, 1, G)
    assert np.array_equal(got_c.cpu().numpy(), want_c)
    want_y = orc.dyn_dilated_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], mode, **kw)
    want_g = orc.dyn_dilated_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, mode, **kw)
    ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
    y = dn.dyn_dilated_conv3d(*ts, mode, 1, 1, 1, 1, G)
    close(y, want_y, dtype, "y")
    y.backward(cu(p["gy"]))
    for t, w_, nm in zip(ts, want_g, ("grad_x", "grad_size_map", "grad_mask", "grad_w", "grad_bias")):
        close(t.grad, w_, dtype, nm)


def test_dyn_dilated_equals_materialised_offsets(dn):
    """Fused field path == reference route (offsets_from_size_map -> deform_conv3d), forward and
    field gradient through autograd."""
    from d2conv3d_b200.dconv_native.grid import offsets_from_size_map
    p = make_problem(201, 2, 4, 6, (3, 6, 6), padding=1, dtype=np.float64, field_mode="xyz")
    ts = [cu(p[k], True) for k in ("x", "geo", "mask", "weight", "bias")]
    y1 = dn.dyn_dilated_conv3d(*ts, "xyz", 1, 1, 1)
    y1.backward(cu(p["gy"]))
    g1 = [t.grad.clone() for t in ts]
    for t in ts:
        t.grad = None
    off = offsets_from_size_map(ts[1], "xyz", (3, 3, 3), (1, 1, 1))
    y2 = dn.deform_conv3d(ts[0], off, ts[2], ts[3], ts[4], 1, 1, 1)
    y2.backward(cu(p["gy"]))
    assert torch.equal(y1, y2)
    for a, t in zip(g1, ts):
        assert torch.allclose(a, t.grad, rtol=1e-9, atol=1e-11)


# ---- packaged layers (ops/dconv-native/test/test_modules.py) --------------------------------------

def test_modules_zero_init_identities(dn):
    torch.manual_seed(1)
    data = torch.randn(2, 3, 7, 7, 7).cuda()
    conv = nn.Conv3d(3, 4, 3).cuda()
    for cls, scale in ((dn.DConv3d, 1.0), (dn.MDConv3d, 0.5)):
        layer = cls(3, 4, 3).cuda()
        layer.deform_conv.weight.data = conv.weight.data
        layer.deform_conv.bias.data = conv.bias.data
        assert torch.allclose(conv(data * scale), layer(data), atol=1e-6)


@pytest.mark.parametrize("fused", [True, False])
def test_size_conditioning_equals_dilated_conv(dn, fused):
    torch.manual_seed(2)
    data = torch.randn(2, 3, 7, 7, 7).cuda()
    conv = nn.Conv3d(3, 4, 3, padding=(1, 2, 2), dilation=(1, 2, 2)).cuda()
    layer = dn.SizeConditionedDConv3d(3, 4, 3, padding=1, fused_field=fused).cuda()
    layer.deform_params.weight.data[0] = 0
    layer.deform_params.bias.data[0] = 1          # size = elu(1) + 1 = 2
    layer.deform_conv.weight.data = conv.weight.data
    layer.deform_conv.bias.data = conv.bias.data
    assert torch.allclose(conv(data), layer(data), atol=1e-6)


def test_module_backward_smoke(dn):
    data = torch.randn(2, 3, 7, 7, 7).cuda()
    layer = dn.XYZSizeConditionedMDConv3d(3, 4, 3, padding=1, bias=False).cuda()
    layer(data).mean().backward()
    assert layer.deform_conv.weight.grad is not None and layer.deform_params.weight.grad is not None
    assert torch.isfinite(layer.deform_params.weight.grad).all()
