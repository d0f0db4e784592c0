"""GPU parity tests of the tensor-core (tcgen05 / TMEM) tier, reached by selecting the
'bf16' math mode: operands (channels-last input, weights, sampled tile) are rounded to
bf16, products accumulate in fp32.  Stated bound for this mode: 1e-2 of the output's
scale (max |y|) against the fp32 oracle, and 2e-3 against the oracle fed bf16-rounded
x and w (what remains is the bf16 rounding of the sampled tile and summation order).
Integer corner indices are the same code as the generic tier (bit-exact, tested there).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests._util import make_problem

pytestmark = pytest.mark.gpu

REL_BF16 = 1e-2
REL_BF16_ROUNDED_INPUTS = 2e-3


@pytest.fixture()
def dn():
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    _lib.lib()
    d2conv3d_b200.set_math_mode("bf16")
    yield dconv_native
    d2conv3d_b200.set_math_mode("auto")
    _lib.device_status()     # raises if any bounded device-side wait gave up


def bf16_round(a):
    return torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()


def cu(a):
    return None if a is None else torch.from_numpy(a).cuda()


CASES = [
    dict(B=1, Cin=64, Cout=64, dims=(4, 8, 8), G=1),                 # 2 full tiles
    dict(B=2, Cin=128, Cout=128, dims=(3, 7, 9), G=2),               # ragged last tile, 2 groups
    dict(B=1, Cin=128, Cout=64, dims=(3, 6, 8), G=1),                # 128 channels per group: 2 slices per tap
    dict(B=1, Cin=64, Cout=512, dims=(2, 8, 9), G=1),                # N = 512: two 256-column MMAs, all of TMEM
    dict(B=1, Cin=64, Cout=320, dims=(2, 8, 9), G=1),                # N = 256 + 64
    dict(B=2, Cin=64, Cout=64, dims=(8, 30, 40), G=1),               # 150 tiles: persistent loop wraps
    dict(B=1, Cin=128, Cout=64, dims=(4, 9, 9), G=2, k=(1, 3, 3), padding=(0, 1, 1)),
    dict(B=1, Cin=64, Cout=64, dims=(5, 9, 9), G=1, stride=(1, 2, 2), dilation=(2, 1, 1), padding=(2, 1, 1)),
]


@pytest.mark.parametrize("ci", range(len(CASES)))
def test_forward_bf16_mode_vs_oracle(dn, ci):
    from d2conv3d_b200 import _lib
    cfg = dict(CASES[ci])
    cfg.setdefault("k", 3)
    cfg.setdefault("padding", 1)
    p = make_problem(300 + ci, dtype=np.float32, offset_std=2.0, **cfg)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=p["offset_groups"])
    n0 = _lib.launch_count()
    _lib.profile_read(); _lib.profile_enable(True)
    y = dn.deform_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), p["stride"],
                         p["padding"], p["dilation"], 1, p["offset_groups"]).cpu().numpy()
    _lib.profile_enable(False)
    phases = [n for n, _ in _lib.profile_read()]
    assert "fwd_sm100_fused" in phases, f"tensor-core tier was not used: {phases}"
    assert _lib.launch_count() - n0 == 4      # input staging, weight staging, sampling records, fused kernel
    want = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
    scale = np.abs(want).max()
    err = np.abs(y - want).max() / scale
    want_r = orc.deform_conv3d_fwd(bf16_round(p["x"]), p["geo"], p["mask"], bf16_round(p["weight"]), p["bias"], **kw)
    err_r = np.abs(y - want_r).max() / scale
    print(f"case {ci}: rel err vs fp32 oracle {err:.3e}, vs bf16-rounded-input oracle {err_r:.3e}")
    assert err <= REL_BF16
    assert err_r <= REL_BF16_ROUNDED_INPUTS


def test_no_mask_no_bias_bf16_mode(dn):
    p = make_problem(320, 1, 64, 64, (3, 8, 8), padding=1, dtype=np.float32, mask=False, bias=False)
    y = dn.deform_conv3d(cu(p["x"]), cu(p["geo"]), None, cu(p["weight"]), None, 1, 1, 1).cpu().numpy()
    want = orc.deform_conv3d_fwd(p["x"], p["geo"], None, p["weight"], None, padding=1)
    assert np.abs(y - want).max() <= REL_BF16 * np.abs(want).max()


@pytest.mark.parametrize("mode", ["x", "xyz"])
def test_dyn_dilated_bf16_mode(dn, mode):
    G = 2
    p = make_problem(330, 2, 128, 64, (4, 9, 10), padding=1, G=G, dtype=np.float32, field_mode=mode)
    y = dn.dyn_dilated_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), mode,
                              1, 1, 1, 1, G).cpu().numpy()
    want = orc.dyn_dilated_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], mode, padding=1,
                                      offset_groups=G)
    assert np.abs(y - want).max() <= REL_BF16 * np.abs(want).max()


def test_unsupported_shapes_fall_back_to_generic_tier(dn):
    """cpg not a multiple of 64 -> CUDA-core kernels even in bf16 mode (still exact fp32 parity)."""
    p = make_problem(340, 1, 48, 32, (3, 6, 6), padding=1, G=2, dtype=np.float32)
    y = dn.deform_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), 1, 1, 1, 1, 2)
    want = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], padding=1, offset_groups=2)
    assert np.abs(y.cpu().numpy() - want).max() <= 1e-4 * np.abs(want).max()


@pytest.mark.parametrize("cfg,bound", [
    (dict(B=2, Cin=256, Cout=128, dims=(2, 6, 9), G=8), REL_BF16),     # units span two offset groups (two record sets)
    (dict(B=1, Cin=64, Cout=64, dims=(3, 7, 8), G=2), REL_BF16),
    (dict(B=1, Cin=96, Cout=192, dims=(3, 6, 8), G=3), 1e-4),          # odd group count: split kernel instead
    (dict(B=1, Cin=64, Cout=512, dims=(2, 6, 8), G=2), 1e-4),          # no room for two record sets: split kernel
])
def test_bf16_mode_with_32_channels_per_group(dn, cfg, bound):
    """32 channels per offset group: a 64-channel single-pass unit then spans two groups and takes chunks 0-3 /
    4-7 of every row from two different record sets; where that does not apply (odd group count, weight slice
    too large to leave room for the second set) bf16 mode runs the split (fp32-parity) kernel."""
    from d2conv3d_b200 import _lib
    p = make_problem(350, padding=1, dtype=np.float32, offset_std=2.0, **cfg)
    _lib.profile_read(); _lib.profile_enable(True)
    y = dn.deform_conv3d(cu(p["x"]), cu(p["geo"]), cu(p["mask"]), cu(p["weight"]), cu(p["bias"]), 1, 1, 1, 1, cfg["G"])
    _lib.profile_enable(False)
    assert "fwd_sm100_fused" in [n for n, _ in _lib.profile_read()]
    want = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], padding=1, offset_groups=cfg["G"])
    err = np.abs(y.cpu().numpy() - want).max() / np.abs(want).max()
    print(cfg, err)
    assert err <= bound
    if bound == REL_BF16:
        assert err > 1e-5, "expected the single-pass kernel (bf16-sized error), got fp32-parity accuracy"


REL_BF16_GRAD = 2e-2


@pytest.mark.parametrize("ci", [0, 1, 2, 3, 6, 7])
def test_backward_bf16_mode_vs_oracle(dn, ci):
    """All five gradients in bf16 mode (tensor-core gradient columns, bf16-staged input) against the fp32
    oracle; bound 2e-2 of each gradient's scale."""
    from d2conv3d_b200 import _lib
    cfg = dict(CASES[ci])
    cfg.setdefault("k", 3)
    cfg.setdefault("padding", 1)
    p = make_problem(400 + ci, dtype=np.float32, offset_std=2.0, **cfg)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=p["offset_groups"])
    want = orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, **kw)
    ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
    y = dn.deform_conv3d(*ts, p["stride"], p["padding"], p["dilation"], 1, p["offset_groups"])
    _lib.profile_read(); _lib.profile_enable(True)
    y.backward(cu(p["gy"]))
    _lib.profile_enable(False)
    phases = [n for n, _ in _lib.profile_read()]
    assert "bwd_dcol_sm100" in phases and "bwd_sample_grad" in phases, phases
    for t, w_, nm in zip(ts, want, ("grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias")):
        err = np.abs(t.grad.cpu().numpy() - w_).max() / np.abs(w_).max()
        print(f"case {ci} {nm}: rel err {err:.3e}")
        assert err <= REL_BF16_GRAD, nm


@pytest.mark.parametrize("mode,G,Cin", [("x", 2, 128), ("xyz", 2, 128), ("xyz", 8, 256)])   # last: 32 channels per group
def test_dyn_dilated_backward_bf16_mode(dn, mode, G, Cin):
    p = make_problem(430, 2, Cin, 64, (4, 9, 10), padding=1, G=G, dtype=np.float32, field_mode=mode)
    want = orc.dyn_dilated_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, mode, padding=1,
                                      offset_groups=G)
    ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
    dn.dyn_dilated_conv3d(*ts, mode, 1, 1, 1, 1, G).backward(cu(p["gy"]))
    for t, w_, nm in zip(ts, want, ("grad_x", "grad_size_map", "grad_mask", "grad_w", "grad_bias")):
        err = np.abs(t.grad.cpu().numpy() - w_).max() / np.abs(w_).max()
        assert err <= REL_BF16_GRAD, (nm, err)


def test_backward_chunked_by_intermediate_cap(dn):
    p = make_problem(440, 3, 64, 64, (2, 8, 9), padding=1, dtype=np.float32)
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
        assert torch.allclose(a, b, rtol=1e-3, atol=1e-4 * float(a.abs().max()))
