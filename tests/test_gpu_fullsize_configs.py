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

Two reference runs per case.  float32 -- the same position arithmetic as this library (integer corners are
bit-identical by construction), so it is the comparator for the gradients w.r.t. offsets / the dilation field, which
jump where a sampling position crosses an integer.  float64 -- the higher-precision arbiter for everything that is
continuous in the position (output, grad_x, grad_mask, grad_w, grad_bias): the reference's own fp32 run carries
rounding noise of the size of this library's.

Bounds.  auto: 1e-4 of each result's scale, and element-wise |a - r| <= 1e-4 |r| + 1e-5 scale.  (The contraction keeps
16 significand bits per operand -- bf16 hi + lo -- and the tensor cores' fp32 accumulator loses about n * 2^-26 of the
result over a chain of n accumulating MMAs, which is why the kernels end a chain after ~650 MMAs and combine partial
results with fp32 atomics; measured worst element 1.6e-5 of scale, worst excess over 1e-4 |r| 7.6e-6 of scale.)
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
    d2conv3d_b200.set_keep_samples(True)
    _lib.device_status()


def _ref():
    ref = _reference.load("dconv_native")
    if ref is None:
        pytest.skip("the reference extension does not import here")
    return ref


FLOOR = 1e-5


def check_all(label, mode, names, got, want32, want64, discontinuous):
    """Prints every tensor's figures, then asserts.  `discontinuous`: names compared with the float32 reference."""
    rows, failures = [], []
    for name, a, r32, r64 in zip(names, got, want32, want64):
        if a is None:
            continue
        r = (r32 if name in discontinuous else r64).double()
        a = a.double()
        scale = float(r.abs().max())
        diff = (a - r).abs()
        worst = float(diff.max()) / max(scale, 1e-30)
        excess = float((diff - 1e-4 * r.abs()).max()) / max(scale, 1e-30)      # what the absolute floor has to cover
        rows.append(f"{label} {mode} {name}: max|a-r|/scale {worst:.2e}, max(|a-r| - 1e-4|r|)/scale {excess:.2e}"
                    f" (vs float{'32' if name in discontinuous else '64'} reference)")
        if mode == "auto":
            if worst > 1e-4:
                failures.append((name, "scale bound", worst))
            if excess > FLOOR:
                failures.append((name, "element-wise bound", excess))
        elif worst > (1e-2 if name == "y" else 2e-2):
            failures.append((name, "bf16-mode bound", worst))
    print("\n".join(rows))
    assert not failures, failures


def run_reference(fn, tensors, gy, dtype):
    """fn(list of leaf tensors) -> output; returns [y, grads...] of the reference in `dtype`."""
    ts = [None if t is None else t.detach().to(dtype).requires_grad_() for t in tensors]
    y = fn(ts)
    y.backward(gy.to(dtype))
    torch.cuda.synchronize()
    return [y.detach()] + [None if t is None else t.grad for t in ts]


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

    def ref_fn(ts):
        offsets = offsets_from_size_map(ts[1], field_mode, (3, 3, 3), (1, 1, 1))
        return ref.deform_conv3d(ts[0], offsets, ts[2], ts[3], ts[4], (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 1)

    tensors = [x, field, mask, w, bias]
    want32 = run_reference(ref_fn, tensors, gy, torch.float32)
    want64 = run_reference(ref_fn, tensors, gy, torch.float64)
    lib_mode(mode)
    got = run_reference(lambda ts: dconv_native.dyn_dilated_conv3d(ts[0], ts[1], ts[2], ts[3], ts[4], field_mode, 1, 1, 1, 1, 1),
                        tensors, gy, torch.float32)
    check_all(f"c3-{field_mode}", mode, ("y", "grad_x", "grad_size_map", "grad_mask", "grad_w", "grad_bias"), got, want32,
              want64, {"grad_size_map"})


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

    def ref_chunked(dtype):
        parts = {k: [] for k in ("y", "gx", "goff", "gmask")}
        gw_ref, gb_ref = torch.zeros_like(w, dtype=dtype), torch.zeros_like(bias, dtype=dtype)
        for b0 in range(0, B, 4):                                   # 4 clips: 1.43e9 column elements < 2^31
            sl = slice(b0, b0 + 4)
            r = run_reference(lambda ts: ref.deform_conv3d(*ts, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, G),
                              [x[sl], off[sl], mask[sl], w, bias], gy[sl], dtype)
            parts["y"].append(r[0]); parts["gx"].append(r[1]); parts["goff"].append(r[2]); parts["gmask"].append(r[3])
            gw_ref += r[4]; gb_ref += r[5]
        return [torch.cat(parts["y"]), torch.cat(parts["gx"]), torch.cat(parts["goff"]), torch.cat(parts["gmask"]),
                gw_ref, gb_ref]

    want32, want64 = ref_chunked(torch.float32), ref_chunked(torch.float64)
    lib_mode(mode)
    got = run_reference(lambda ts: dconv_native.deform_conv3d(*ts, (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, G),
                        [x, off, mask, w, bias], gy, torch.float32)
    check_all("c4-md", mode, ("y", "grad_x", "grad_offset", "grad_mask", "grad_w", "grad_bias"), got, want32, want64,
              {"grad_offset"})


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

    def ref_fn(ts):
        offsets = offsets_from_size_map(ts[1], "xyz", (3, 3, 3), (1, 1, 1)).repeat(1, G, 1, 1, 1)
        return ref.deform_conv3d(ts[0], offsets, ts[2], ts[3], ts[4], (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, G)

    tensors = [x, field, mask, w, bias]
    want32 = run_reference(ref_fn, tensors, gy, torch.float32)
    want64 = run_reference(ref_fn, tensors, gy, torch.float64)
    lib_mode(mode)
    got = run_reference(lambda ts: dconv_native.dyn_dilated_conv3d(*ts, "xyz", 1, 1, 1, 1, G), tensors, gy, torch.float32)
    check_all("c5-e1", mode, ("y", "grad_x", "grad_size_map", "grad_mask", "grad_w", "grad_bias"), got, want32, want64,
              {"grad_size_map"})


# ---- many tiles through the 32-channels-per-group kernel variants -------------------------------------------------

_oracle_cache = {}


def _many_tile_case(kind):
    """B=2, 128->128 channels in 4 offset groups of 32, 6x40x80: 2 x 19 200 voxels = 300 tiles of 128.  The oracle
    runs in float32 (same position arithmetic: the offset / field gradients jump at integer positions) and in
    float64 (arbiter for the continuous results)."""
    if kind not in _oracle_cache:
        G = 4
        p = make_problem(1900, 2, 128, 128, (6, 40, 80), padding=1, G=G, dtype=np.float32, offset_std=2.0,
                         field_mode="xyz" if kind == "field" else None)
        kw = dict(stride=1, padding=1, dilation=1, groups=1, offset_groups=G)
        res = {}
        for dt in (np.float32, np.float64):
            d = lambda k: p[k].astype(dt)
            if kind == "field":
                y = orc.dyn_dilated_conv3d_fwd(d("x"), d("geo"), d("mask"), d("weight"), d("bias"), "xyz", **kw)
                g = orc.dyn_dilated_conv3d_bwd(d("gy"), d("x"), d("geo"), d("mask"), d("weight"), True, "xyz", **kw)
            else:
                y = orc.deform_conv3d_fwd(d("x"), d("geo"), d("mask"), d("weight"), d("bias"), **kw)
                g = orc.deform_conv3d_bwd(d("gy"), d("x"), d("geo"), d("mask"), d("weight"), True, **kw)
            res[dt] = [torch.from_numpy(np.asarray(a)) for a in (y,) + tuple(g)]
        _oracle_cache[kind] = (p, res[np.float32], res[np.float64])
    return _oracle_cache[kind]


@pytest.mark.parametrize("keep", [False, True])
@pytest.mark.parametrize("kind", ["offsets", "field"])
@pytest.mark.parametrize("mode", ["auto", "bf16"])
def test_300_tiles_with_32_channels_per_offset_group(lib_mode, mode, kind, keep):
    """auto: split forward on 32-channel units, sampling gradient on half slices, weight gradient from two groups'
    records per slice.  bf16: forward and weight gradient with two record sets per ring stage.  keep: the weight
    gradient streams the samples the forward kept instead of gathering them again (the default for training)."""
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    p, want32, want64 = _many_tile_case(kind)
    lib_mode(mode)
    d2conv3d_b200.set_keep_samples(keep)
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
    d2conv3d_b200.set_keep_samples(True)
    assert {"fwd_sm100_fused", "bwd_dcol_sm100", "bwd_sample_grad",
            "bwd_dw_sm100_saved" if keep else "bwd_dw_sm100"} <= phases, phases
    got = [y.detach().cpu()] + [t.grad.cpu() for t in ts]
    check_all(f"300-tiles-{kind}", mode, ("y", "grad_x", "grad_geo", "grad_mask", "grad_w", "grad_bias"), got, want32, want64,
              {"grad_geo"})
