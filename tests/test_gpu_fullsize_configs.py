"""Full-size parity of the secondary benchmark configurations against the reference's own compiled CUDA op
(baseline/_ref, unmodified sources), forward and every gradient, in the fp32-parity mode ("auto") and the
single-pass "bf16" mode:

  C3     dynamic-dilation conv3d, B=4, 256->256, 8x60x108, modes xyz / xy / x, optional 27-channel mask.  The
         reference has no field op: it is fed offsets_from_size_map(field) (utils/grid.py:72-98) and autograd
         carries its grad_offset back to the field.
  C4-MD  modulated deformable 1024->256, B=8, 8x30x54, G=8.  B*Cin*K*V = 2.87e9 overflows the reference's 32-bit
         element count (csrc/ops/dconv3d_gpu.cu:536-553), so the reference runs in two chunks of 4 clips.
  C5-e1  the decoder's stride-4 layer: xyz field + per-group masks, 256->256, 8x120x214, G=8 (32 channels per offset
         group), one clip.  The reference needs one offset set per group: the shared field's offsets repeated G
         times (`offsets.repeat(1, G, 1, 1, 1)`).

plus many-tile cases (300 tiles) of every kernel variant that serves 32 channels per offset group, against the CPU
oracle, so that their persistent loops, ring wrap-around and partial-tile reductions run under a test.

Bounds.  auto: 1e-4 of each result's scale AND an element-wise mixed bound |a - r| <= 1e-4 |r| + 1e-5 scale.
bf16: output 1e-2, gradients 2e-2 of scale (the stated bound of that mode).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import _reference
from tests._util import make_problem

pytestmark = pytest.mark.gpu

needs_ref = pytest.mark.skipif(not _reference.available(), reason="baseline/_ref (the reference's compiled op) is absent")


@pytest.fixture()
def lib_mode():
    import d2conv3d_b200
    from d2conv3d_b200 import _lib
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False

    def set_mode(m):
        d2conv3d_b200.set_math_mode(m)
    yield set_mode
    d2conv3d_b200.set_math_mode("auto")
    _lib.device_status()


def _ref():
    ref = _reference.load("dconv_native")
    if ref is None:
        pytest.skip("the reference extension does not import here")
    return ref


def check(name, got, want, mode, is_output=False):
    got, want = got.float(), want.float()
    scale = float(want.abs().max())
    diff = (got - want).abs()
    worst = float(diff.max()) / max(scale, 1e-30)
    if mode == "auto":
        assert worst <= 1e-4, (name, worst)
        excess = diff - (1e-4 * want.abs() + 1e-5 * scale)
        assert float(excess.max()) <= 0, (name, "element-wise mixed bound", float(excess.max()), scale)
    else:
        assert worst <= (1e-2 if is_output else 2e-2), (name, worst)
    return worst


def seeded(seed, *shapes):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(s, generator=g) for s in shapes]


# ---- C3: dilation field ---------------------------------------------------------------------------------------

@needs_ref
@pytest.mark.parametrize("field_mode,nch", [("xyz", 3), ("xy", 2), ("x", 1)])
@pytest.mark.parametrize("mode", ["auto", "bf16"])
def test_c3_field_full_size_vs_reference(lib_mode, mode, field_mode, nch):
    from d2conv3d_b200 import dconv_native
    from d2conv3d_b200.dconv_native.grid import offsets_from_size_map
    ref = _ref()
    B, C, dims = 4, 256, (8, 60, 108)
    x, f, m, w, gy = seeded(1003, (B, C) + dims, (B, nch) + dims, (B, 27) + dims, (C, C, 3, 3, 3), (B, C) + dims)
    field = (1 + torch.nn.functional.softplus(f)).cuda()
    x, w, gy = x.cuda(), (w * (2.0 / (C * 27)) ** 0.5).cuda(), gy.cuda()
    mask = torch.sigmoid(m).cuda() if field_mode == "xyz" else None        # "optional modulation mask": with and without
    bias = torch.zeros(C, device="cuda")

    ts = [t.detach().clone().requires_grad_() for t in (x, field, w, bias)]
    mk = None if mask is None else mask.detach().clone().requires_grad_()
    offsets = offsets_from_size_map(ts[1], field_mode, (3, 3, 3), (1, 1, 1))
    y_ref = ref.deform_conv3d(ts[0], offsets, mk, ts[2], ts[3], (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 1)
    y_ref.backward(gy)
    torch.cuda.synchronize()
    want = [y_ref.detach(), ts[0].grad, ts[1].grad, ts[2].grad, ts[3].grad, None if mk is None else mk.grad]
    del offsets, y_ref

    lib_mode(mode)
    us = [t.detach().clone().requires_grad_() for t in (x, field, w, bias)]
    mk2 = None if mask is None else mask.detach().clone().requires_grad_()
    y = dconv_native.dyn_dilated_conv3d(us[0], us[1], mk2, us[2], us[3], field_mode, 1, 1, 1, 1, 1)
    y.backward(gy)
    torch.cuda.synchronize()
    got = [y.detach(), us[0].grad, us[1].grad, us[2].grad, us[3].grad, None if mk2 is None else mk2.grad]
    for name, a, r in zip(("y", "grad_x", "grad_size_map", "grad_w", "grad_bias", "grad_mask"), got, want):
        if r is not None:
            print(f"c3-{field_mode} {mode} {name}: {check(name, a, r, mode, name == 'y'):.2e}")


# ---- C4-MD ------------------------------------------------------------------------------------------------------

@needs_ref
@pytest.mark.parametrize("mode", ["auto", "bf16"])
def test_c4_md_full_size_vs_reference_in_two_chunks(lib_mode, mode):
    from d2conv3d_b200 import dconv_native
    ref = _ref()
    B, Cin, Cout, dims, G = 8, 1024, 256, (8, 30, 54), 8
    x, o, m, w, gy = seeded(1004, (B, Cin) + dims, (B, G * 81) + dims, (B, G * 27) + dims, (Cout, Cin, 3, 3, 3),
                            (B, Cout) + dims)
    x, off, mask, gy = x.cuda(), (o * 2.0).cuda(), torch.sigmoid(m).cuda(), gy.cuda()
    w = (w * (2.0 / (Cin * 27)) ** 0.5).cuda()
    bias = torch.zeros(Cout, device="cuda")

    want = {k: [] for k in ("y", "gx", "goff", "gmask")}
    gw_ref, gb_ref = torch.zeros_like(w), torch.zeros_like(bias)
    for b0 in range(0, B, 4):                                   # 4 clips: 1.43e9 column elements < 2^31
        sl = slice(b0, b0 + 4)
        ts = [t.detach().clone().requires_grad_() for t in (x[sl], off[sl], mask[sl], w, bias)]
        y_ref = ref.deform_conv3d(*ts, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, G)
        y_ref.backward(gy[sl])
        torch.cuda.synchronize()
        want["y"].append(y_ref.detach()); want["gx"].append(ts[0].grad); want["goff"].append(ts[1].grad)
        want["gmask"].append(ts[2].grad)
        gw_ref += ts[3].grad; gb_ref += ts[4].grad
        del y_ref, ts
    lib_mode(mode)
    us = [t.detach().clone().requires_grad_() for t in (x, off, mask, w, bias)]
    y = dconv_native.deform_conv3d(*us, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, G)
    y.backward(gy)
    torch.cuda.synchronize()
    pairs = [("y", y.detach(), torch.cat(want["y"])), ("grad_x", us[0].grad, torch.cat(want["gx"])),
             ("grad_offset", us[1].grad, torch.cat(want["goff"])), ("grad_mask", us[2].grad, torch.cat(want["gmask"])),
             ("grad_w", us[3].grad, gw_ref), ("grad_bias", us[4].grad, gb_ref)]
    for name, a, r in pairs:
        print(f"c4-md {mode} {name}: {check(name, a, r, mode, name == 'y'):.2e}")


# ---- C5 stride-4 layer: shared field, 8 groups of 32 channels -----------------------------------------------------

@needs_ref
@pytest.mark.parametrize("mode", ["auto", "bf16"])
def test_c5_e1_layer_full_size_vs_reference_with_repeated_offsets(lib_mode, mode):
    from d2conv3d_b200 import dconv_native
    from d2conv3d_b200.dconv_native.grid import offsets_from_size_map
    ref = _ref()
    B, C, dims, G = 1, 256, (8, 120, 214), 8
    x, f, m, w, gy = seeded(1005, (B, C) + dims, (B, 3) + dims, (B, G * 27) + dims, (C, C, 3, 3, 3), (B, C) + dims)
    x, gy = torch.relu(x).cuda(), gy.cuda()
    field, mask = (1 + torch.nn.functional.softplus(f)).cuda(), torch.sigmoid(m).cuda()
    w = (w * (2.0 / (C * 27)) ** 0.5).cuda()
    bias = torch.zeros(C, device="cuda")

    ts = [t.detach().clone().requires_grad_() for t in (x, field, mask, w, bias)]
    offsets = offsets_from_size_map(ts[1], "xyz", (3, 3, 3), (1, 1, 1)).repeat(1, G, 1, 1, 1)
    y_ref = ref.deform_conv3d(ts[0], offsets, ts[2], ts[3], ts[4], (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, G)
    y_ref.backward(gy)
    torch.cuda.synchronize()
    want = [y_ref.detach()] + [t.grad for t in ts]
    del offsets, y_ref

    lib_mode(mode)
    us = [t.detach().clone().requires_grad_() for t in (x, field, mask, w, bias)]
    y = dconv_native.dyn_dilated_conv3d(*us, "xyz", 1, 1, 1, 1, G)
    y.backward(gy)
    torch.cuda.synchronize()
    got = [y.detach()] + [t.grad for t in us]
    for name, a, r in zip(("y", "grad_x", "grad_size_map", "grad_mask", "grad_w", "grad_bias"), got, want):
        print(f"c5-e1 {mode} {name}: {check(name, a, r, mode, name == 'y'):.2e}")


# ---- many tiles through the 32-channels-per-group kernel variants -------------------------------------------------

_oracle_cache = {}


def _many_tile_case(kind):
    """B=2, 128->128 channels in 4 offset groups of 32, 6x40x80: 2 x 19 200 voxels = 300 tiles of 128."""
    if kind not in _oracle_cache:
        G = 4
        p = make_problem(1900, 2, 128, 128, (6, 40, 80), padding=1, G=G, dtype=np.float32, offset_std=2.0,
                         field_mode="xyz" if kind == "field" else None)
        kw = dict(stride=1, padding=1, dilation=1, groups=1, offset_groups=G)
        if kind == "field":
            y = orc.dyn_dilated_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], "xyz", **kw)
            g = orc.dyn_dilated_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, "xyz", **kw)
        else:
            y = orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
            g = orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, **kw)
        _oracle_cache[kind] = (p, y, g)
    return _oracle_cache[kind]


@pytest.mark.parametrize("kind", ["offsets", "field"])
@pytest.mark.parametrize("mode", ["auto", "bf16"])
def test_300_tiles_with_32_channels_per_offset_group(lib_mode, mode, kind):
    """auto: split forward on 32-channel units, sampling gradient on half slices, weight gradient from two groups'
    records per slice.  bf16: forward and weight gradient with two record sets per ring stage."""
    from d2conv3d_b200 import _lib, dconv_native
    p, want_y, want_g = _many_tile_case(kind)
    lib_mode(mode)
    cu = lambda a: torch.from_numpy(a).cuda()
    ts = [cu(p[k]).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
    _lib.profile_read(); _lib.profile_enable(True)
    if kind == "field":
        y = dconv_native.dyn_dilated_conv3d(*ts, "xyz", 1, 1, 1, 1, 4)
    else:
        y = dconv_native.deform_conv3d(*ts, 1, 1, 1, 1, 4)
    y.backward(cu(p["gy"]))
    _lib.profile_enable(False)
    phases = {n for n, _ in _lib.profile_read()}
    assert {"fwd_sm100_fused", "bwd_dcol_sm100", "bwd_sample_grad", "bwd_dw_sm100"} <= phases, phases
    print(f"{kind} {mode} y: {check('y', y.detach().cpu(), torch.from_numpy(want_y), mode, True):.2e}")
    for name, t, r in zip(("grad_x", "grad_geo", "grad_mask", "grad_w", "grad_bias"), ts, want_g):
        print(f"{kind} {mode} {name}: {check(name, t.grad.cpu(), torch.from_numpy(r), mode):.2e}")
