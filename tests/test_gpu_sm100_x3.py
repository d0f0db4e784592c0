"""GPU parity tests of the tensor-core tier in its fp32-parity mode ('bf16x3', also what 'auto' selects
where the tensor-core kernels apply): every fp32 operand is split into bf16 hi + lo, the contraction is
a_hi*b_hi + a_lo*b_hi + a_hi*b_lo with fp32 accumulation, the trilinear blend is done in fp32 on fp32
channels-last data.  Bound: the same 1e-4 of the result's scale as the exact fp32 tier (the reference's
cuBLAS fp32 GEMM and this split differ by ~1e-5)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests._util import make_problem

pytestmark = pytest.mark.gpu

REL = 1e-4


@pytest.fixture(params=["bf16x3", "auto"])
def dn(request):
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    _lib.lib()
    d2conv3d_b200.set_math_mode(request.param)
    yield dconv_native
    d2conv3d_b200.set_math_mode("auto")
    _lib.device_status()     # raises if any bounded device-side wait gave up


def cu(a):
    return None if a is None else torch.from_numpy(a).cuda()


CASES = [
    dict(B=1, Cin=64, Cout=64, dims=(4, 8, 8), G=1),                 # 2 full tiles
    dict(B=2, Cin=128, Cout=128, dims=(3, 7, 9), G=2),               # ragged last tile, 2 groups
    dict(B=1, Cin=128, Cout=64, dims=(3, 6, 8), G=1),                # 128 channels per group: 4 units per tap
    dict(B=1, Cin=64, Cout=512, dims=(2, 8, 9), G=1),                # N = 512: two 256-column MMAs, all of TMEM
    dict(B=1, Cin=64, Cout=320, dims=(2, 8, 9), G=1),                # N = 256 + 64
    dict(B=2, Cin=64, Cout=64, dims=(8, 30, 40), G=1),               # 150 tiles: persistent loop wraps
    dict(B=1, Cin=128, Cout=64, dims=(4, 9, 9), G=2, k=(1, 3, 3), padding=(0, 1, 1)),
    dict(B=1, Cin=64, Cout=64, dims=(5, 9, 9), G=1, stride=(1, 2, 2), dilation=(2, 1, 1), padding=(2, 1, 1)),
]


@pytest.mark.parametrize("ci", range(len(CASES)))
def test_forward_fp32_parity_mode_vs_oracle(dn, ci):
    from d2conv3d_b200 import _lib
    cfg = dict(CASES[ci])
    cfg.setdefault("k", 3)
    cfg.setdefault("padding", 1)
    p = make_problem(700 + ci, dtype=np.float32, offset_std=2.0, **cfg)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=p["offset_groups"])
    _lib.profile_read(); _lib.profile_enable(True)
    y = dn.deform_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), p["stride"],
                         p["padding"], p["dilation"], 1, p["offset_groups"]).cpu().numpy()
    _lib.profile_enable(False)
    phases = [n for n, _ in _lib.profile_read()]
    assert "fwd_sm100_fused" in phases, f"tensor-core tier was not used: {phases}"
    want = orc.deform_conv3d_fwd(p["x"].astype(np.float64), p["geo"].astype(np.float64), p["mask"].astype(np.float64),
                                 p["weight"].astype(np.float64), p["bias"].astype(np.float64), **kw)
    err = np.abs(y - want).max() / np.abs(want).max()
    print(f"case {ci}: rel err vs float64 oracle {err:.3e}")
    assert err <= REL


@pytest.mark.parametrize("cfg", [dict(B=1, Cin=64, Cout=64, dims=(3, 7, 8), G=2),
                                 dict(B=2, Cin=256, Cout=256, dims=(2, 6, 9), G=8)])
def test_forward_32_channels_per_offset_group(dn, cfg):
    """32 channels per offset group (e.g. 256 channels in 8 groups): a 32-channel unit of the fp32-parity mode
    still lies inside one group, so the forward stays on the tensor cores."""
    from d2conv3d_b200 import _lib
    p = make_problem(760, dtype=np.float32, offset_std=2.0, k=3, padding=1, **cfg)
    _lib.profile_read(); _lib.profile_enable(True)
    y = dn.deform_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), 1, 1, 1, 1,
                         cfg["G"]).cpu().numpy()
    _lib.profile_enable(False)
    assert "fwd_sm100_fused" in [n for n, _ in _lib.profile_read()]
    want = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], padding=1, offset_groups=cfg["G"])
    assert np.abs(y - want).max() <= REL * np.abs(want).max()
    # the backward of such a shape runs on the generic tier and must still be right
    ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
    dn.deform_conv3d(*ts, 1, 1, 1, 1, cfg["G"]).backward(cu(p["gy"]))
    wantg = orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, padding=1,
                                  offset_groups=cfg["G"])
    for t, w_ in zip(ts, wantg):
        assert np.abs(t.grad.cpu().numpy() - w_).max() <= REL * np.abs(w_).max()


def test_integer_and_border_coordinates(dn):
    """Offsets that put samples exactly on voxels, on the -1 / size borders and far outside: the clamped
    stand-in corners must contribute exactly nothing."""
    p = make_problem(720, 1, 64, 64, (3, 6, 7), padding=1, dtype=np.float32, offset_std=0.0)
    rng = np.random.default_rng(5)
    p["geo"][:] = rng.integers(-4, 5, size=p["geo"].shape).astype(np.float32)
    y = dn.deform_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), 1, 1, 1).cpu().numpy()
    want = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], padding=1)
    assert np.abs(y - want).max() <= REL * np.abs(want).max()


@pytest.mark.parametrize("mode", ["x", "xyz"])
def test_dyn_dilated_fp32_parity_mode(dn, mode):
    G = 2
    p = make_problem(730, 2, 128, 64, (4, 9, 10), padding=1, G=G, dtype=np.float32, field_mode=mode)
    y = dn.dyn_dilated_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), mode,
                              1, 1, 1, 1, G).cpu().numpy()
    want = orc.dyn_dilated_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], mode, padding=1,
                                      offset_groups=G)
    assert np.abs(y - want).max() <= REL * np.abs(want).max()


@pytest.mark.parametrize("ci", [0, 1, 2, 3, 4, 6, 7])
def test_backward_fp32_parity_mode_vs_oracle(dn, ci):
    """All five gradients on the tensor-core tier in the fp32-parity mode against the float64 oracle; 1e-4 of
    each gradient's scale (case 3: Cout = 512, the gradient-column contraction runs as two launches
    into two partial buffers; case 4: Cout = 320, a partial second launch)."""
    from d2conv3d_b200 import _lib
    cfg = dict(CASES[ci])
    cfg.setdefault("k", 3)
    cfg.setdefault("padding", 1)
    p = make_problem(800 + ci, dtype=np.float32, offset_std=2.0, **cfg)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=p["offset_groups"])
    d = lambda k: p[k].astype(np.float64)
    want = orc.deform_conv3d_bwd(d("gy"), d("x"), d("geo"), d("mask"), d("weight"), True, **kw)
    ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
    y = dn.deform_conv3d(*ts, p["stride"], p["padding"], p["dilation"], 1, p["offset_groups"])
    _lib.profile_read(); _lib.profile_enable(True)
    y.backward(cu(p["gy"]))
    _lib.profile_enable(False)
    phases = [n for n, _ in _lib.profile_read()]
    assert "bwd_dcol_sm100" in phases and "bwd_sample_grad" in phases, phases
    assert "bwd_dw_sm100" in phases or "bwd_dw_sm100_saved" in phases, phases
    for t, w_, nm in zip(ts, want, ("grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")):
        err = np.abs(t.grad.cpu().numpy() - w_).max() / np.abs(w_).max()
        print(f"case {ci} {nm}: rel err {err:.3e}")
        assert err <= REL, nm


@pytest.mark.parametrize("mode", ["x", "xyz"])
def test_dyn_dilated_backward_fp32_parity_mode(dn, mode):
    G = 2
    p = make_problem(830, 2, 128, 64, (4, 9, 10), padding=1, G=G, dtype=np.float32, field_mode=mode)
    want = orc.dyn_dilated_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, mode, padding=1,
                                      offset_groups=G)
    ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
    dn.dyn_dilated_conv3d(*ts, mode, 1, 1, 1, 1, G).backward(cu(p["gy"]))
    for t, w_, nm in zip(ts, want, ("grad_x", "grad_size_map", "grad_mask", "grad_w", "grad_bias")):
        err = np.abs(t.grad.cpu().numpy() - w_).max() / np.abs(w_).max()
        assert err <= REL, (nm, err)


def test_backward_chunked_by_intermediate_cap_fp32_parity_mode(dn):
    p = make_problem(840, 3, 64, 64, (2, 8, 9), padding=1, dtype=np.float32)
    def run():
        ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
        dn.deform_conv3d(*ts, 1, 1, 1, 1, 1).backward(cu(p["gy"]))
        return [t.grad.clone() for t in ts]
    full = run()
    old = dn._ops.config.get_max_intermediate_elements()
    try:
        dn._ops.config.set_max_intermediate_elements(64 * 27 * 144)    # one clip per chunk
        chunked = run()
    finally:
        dn._ops.config.set_max_intermediate_elements(old)
    for a, b in zip(full, chunked):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5 * float(a.abs().max()))


@pytest.mark.parametrize("cfg", [
    dict(B=2, Cin=256, Cout=128, dims=(2, 6, 9), G=8),      # the decoder's refine-block convs: 8 groups of 32
    dict(B=1, Cin=64, Cout=64, dims=(3, 7, 8), G=2),
    dict(B=2, Cin=128, Cout=512, dims=(2, 5, 6), G=4, stride=(1, 2, 1), dilation=(1, 1, 2)),   # two dcol launches
])
@pytest.mark.parametrize("tc_mode", ["auto", "bf16"])
def test_backward_32_channels_per_offset_group(tc_mode, cfg):
    """32 channels per offset group (even group count): the backward keeps 64-channel slices, each spanning two
    neighbouring groups -- the sampling-gradient kernel serves one group per block on its half of the slice, the
    weight-gradient kernel takes the two halves of a slice from the two groups' records.  fp32-parity mode: 1e-4;
    `bf16` mode: its 2e-2 (single-pass kernels with two record sets per stage up to Cout = 256, the fp32-parity
    kernels above that)."""
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    cfg = dict(cfg)
    cfg.setdefault("padding", 1)
    p = make_problem(860, dtype=np.float32, offset_std=2.0, **cfg)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=cfg["G"])
    d = lambda k: p[k].astype(np.float64)
    want = orc.deform_conv3d_bwd(d("gy"), d("x"), d("geo"), d("mask"), d("weight"), True, **kw)
    d2conv3d_b200.set_math_mode(tc_mode)
    try:
        ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
        y = dconv_native.deform_conv3d(*ts, p["stride"], p["padding"], p["dilation"], 1, cfg["G"])
        _lib.profile_read(); _lib.profile_enable(True)
        y.backward(cu(p["gy"]))
        _lib.profile_enable(False)
        _lib.device_status()
    finally:
        d2conv3d_b200.set_math_mode("auto")
    phases = [n for n, _ in _lib.profile_read()]
    assert "bwd_dcol_sm100" in phases and "bwd_sample_grad" in phases, phases
    assert "bwd_dw_sm100" in phases or "bwd_dw_sm100_saved" in phases, phases
    for t, w_, nm in zip(ts, want, ("grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")):
        err = np.abs(t.grad.cpu().numpy() - w_).max() / np.abs(w_).max()
        print(f"{cfg} {tc_mode} {nm}: rel err {err:.3e}")
        assert err <= (REL if tc_mode == "auto" else 2e-2), nm


def test_dyn_dilated_backward_32_channels_per_offset_group(dn):
    G = 8
    p = make_problem(870, 1, 256, 64, (3, 6, 8), padding=1, G=G, dtype=np.float32, field_mode="xyz")
    want = orc.dyn_dilated_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, "xyz", padding=1,
                                      offset_groups=G)
    from d2conv3d_b200 import _lib
    ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
    y = dn.dyn_dilated_conv3d(*ts, "xyz", 1, 1, 1, 1, G)
    _lib.profile_read(); _lib.profile_enable(True)
    y.backward(cu(p["gy"]))
    _lib.profile_enable(False)
    assert "bwd_dcol_sm100" in [n for n, _ in _lib.profile_read()]
    for t, w_, nm in zip(ts, want, ("grad_x", "grad_size_map", "grad_mask", "grad_w", "grad_bias")):
        err = np.abs(t.grad.cpu().numpy() - w_).max() / np.abs(w_).max()
        assert err <= REL, (nm, err)
