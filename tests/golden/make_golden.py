"""Generates the golden fixtures in this folder from the reference's own Python code.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference [size_map] [deform3d] [deform1d]

(no set names: all three sets).

What it executes from the reference (imported as modules, nothing is copied):
  * ops/dconv-native/test/test_deform_conv.py : `expected_fn` -- the reference's
    executable forward specification (pure Python, float64), run on seeded inputs
    for each geometry its DeformConv3dTester uses plus a few edge cases
    (integer / exactly -1 coordinates, 1x1x1 kernel, mask of ones).
  * utils/grid.py and ops/dconv-native/src/dconv_native/grid.py :
    `offsets_from_size_map` -- dilation field -> offsets, every mode, float32 and
    float64, including the field == 1 case (offset exactly 0).

The test module imports the compiled `dconv_native` extension at import time and
`utils/grid.py` imports `utils.util` (which needs imageio); both are satisfied by
stub modules because only the pure-Python functions are wanted.

  * the same `expected_fn` with N = 1 (linear interpolation) for the geometries of DeformConv1dTester
    (:232-340) plus integer offsets.

Outputs: deform_fwd_cases.npz, size_map_cases.npz, deform1d_fwd_cases.npz (a few hundred KB in total).
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch
from torch.nn.modules.utils import _triple

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py <path of the reference checkout>")
REF = sys.argv[1]


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_reference_test_module():
    stub = types.ModuleType("dconv_native")
    stub.deform_conv1d = stub.deform_conv3d = None
    sys.modules["dconv_native"] = stub
    return _load(os.path.join(REF, "ops/dconv-native/test/test_deform_conv.py"), "_ref_test_deform_conv")


def load_reference_grids():
    utils_pkg = types.ModuleType("utils")
    utils_util = types.ModuleType("utils.util")
    utils_util._triple = _triple
    sys.modules["utils"], sys.modules["utils.util"] = utils_pkg, utils_util
    new = _load(os.path.join(REF, "utils/grid.py"), "_ref_utils_grid")
    old = _load(os.path.join(REF, "ops/dconv-native/src/dconv_native/grid.py"), "_ref_dconv_grid")
    return new, old


# name -> generate_data kwargs (the geometries of DeformConv3dTester,
# ops/dconv-native/test/test_deform_conv.py:343-505) + extra call kwargs
CASES = {
    "default": dict(),
    "stride3": dict(stride=3),
    "offset_groups": dict(channels_in=6, channels_out=4, n_offset_groups=2),
    "weight_groups": dict(channels_in=12, channels_out=6, n_weight_groups=3),
    "groups": dict(channels_in=24, channels_out=12, n_weight_groups=6, n_offset_groups=2),
    "channel_sep_groups": dict(channels_in=6, channels_out=6, n_weight_groups=6, n_offset_groups=3),
    "forward_mixed": dict(batch_size=2, channels_in=2, channels_out=3, dimensions=(5, 7, 7),
                          kernel_size=(3, 3, 3), stride=(1, 2, 1), padding=(0, 1, 2), dilation=(1, 1, 2)),
    "large_batch": dict(batch_size=21, channels_in=2, channels_out=2, dimensions=(3, 5, 5),
                        kernel_size=(1, 3, 3)),
    "backward_geom": dict(batch_size=2, channels_in=3, channels_out=5, dimensions=(2, 3, 5),
                          kernel_size=(3, 5, 3), stride=(1, 2, 1), padding=(1, 3, 5), dilation=(1, 1, 2)),
    "no_bias": dict(bias=False),
    # extra edge cases
    "pad1_big_offsets": dict(channels_in=4, channels_out=4, dimensions=(4, 6, 6), padding=1,
                             n_offset_groups=2, _offset_scale=3.0),
    "pad1_integer_offsets": dict(channels_in=2, channels_out=2, dimensions=(4, 5, 5), padding=1,
                                 _integer_offsets=True),
    "pad1_zero_offsets": dict(channels_in=2, channels_out=2, dimensions=(4, 5, 5), padding=1,
                              _zero_offsets=True),
    "k1": dict(channels_in=4, channels_out=3, dimensions=(3, 4, 5), kernel_size=1),
    "ones_mask": dict(_ones_mask=True),
}


def make_deform_cases():
    ref = load_reference_test_module()
    out = {}
    names = []
    for idx, (name, kw) in enumerate(CASES.items()):
        kw = dict(kw)
        torch.manual_seed(1234 + idx)
        scale = kw.pop("_offset_scale", None)
        integer = kw.pop("_integer_offsets", False)
        zero = kw.pop("_zero_offsets", False)
        ones_mask = kw.pop("_ones_mask", False)
        x, offset, alpha, weight, bias = ref.generate_data(3, device="cpu", dtype=torch.float64, **kw)
        if scale:
            offset = offset * scale
        if integer:
            offset = torch.randint(-2, 3, offset.shape).to(torch.float64)
        if zero:
            offset = torch.zeros_like(offset)
        if ones_mask:
            alpha = torch.ones_like(alpha)
        stride = kw.get("stride", 1)
        padding = kw.get("padding", 0)
        dilation = kw.get("dilation", 1)
        expected = ref.expected_fn(3, x, offset, alpha, weight, bias, stride, padding, dilation)
        names.append(name)
        out[f"{name}/x"] = x.numpy()
        out[f"{name}/offset"] = offset.numpy()
        out[f"{name}/mask"] = alpha.numpy()
        out[f"{name}/weight"] = weight.numpy()
        if bias is not None:
            out[f"{name}/bias"] = bias.numpy()
        out[f"{name}/expected"] = expected.numpy()
        out[f"{name}/geom"] = np.array(
            list(_triple(stride)) + list(_triple(padding)) + list(_triple(dilation))
            + [kw.get("n_weight_groups", 1), kw.get("n_offset_groups", 1)], dtype=np.int64)
        print(f"{name}: out {tuple(expected.shape)}", flush=True)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "deform_fwd_cases.npz"), **out)


def make_size_map_cases():
    new, old = load_reference_grids()
    out = {}
    names = []
    geoms = [((3, 3, 3), (1, 1, 1)), ((3, 3, 3), (1, 2, 2)), ((1, 3, 3), (1, 1, 1)),
             ((3, 5, 3), (2, 1, 3)), ((2, 4, 2), (1, 1, 1))]
    torch.manual_seed(4321)
    for dt in (torch.float32, torch.float64):
        for gi, (k, dil) in enumerate(geoms):
            for mode, nch in (("x", 1), ("xy", 2), ("xxz", 2), ("xyz", 3)):
                size_map = 1 + torch.nn.functional.softplus(torch.randn(2, nch, 3, 4, 5, dtype=dt))
                size_map[0, :, 0, 0, :] = 1.0      # offset exactly zero
                size_map[1, :, 1, 1, :] = 2.0
                size_map[1, :, 2, :, 0] = 0.25     # shrinking field
                off = new.offsets_from_size_map(size_map, mode, k, dil)
                name = f"{mode}_g{gi}_{'f32' if dt == torch.float32 else 'f64'}"
                names.append(name)
                out[f"{name}/size_map"] = size_map.numpy()
                out[f"{name}/offsets"] = off.numpy()
                out[f"{name}/kd"] = np.array(list(k) + list(dil), dtype=np.int64)
                if mode in ("x", "xy", "xyz"):
                    # the older copy shipped inside dconv_native infers the mode from the channel count
                    off_old = old.offsets_from_size_map(size_map, k, dil)
                    assert torch.equal(off, off_old), name
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "size_map_cases.npz"), **out)
    print(f"size-map cases: {len(names)}")


# geometries of DeformConv1dTester (ops/dconv-native/test/test_deform_conv.py:232-340) + integer offsets
CASES_1D = {
    "default": dict(),
    "stride3": dict(stride=3),
    "offset_groups": dict(channels_in=12, channels_out=4, n_offset_groups=2, bias=False),
    "weight_groups": dict(channels_in=12, channels_out=6, n_weight_groups=3, bias=False),
    "groups": dict(channels_in=24, channels_out=12, n_weight_groups=6, n_offset_groups=2, bias=False),
    "forward_mixed": dict(batch_size=3, channels_in=3, channels_out=5, dimensions=34, kernel_size=5, stride=2,
                          padding=3, dilation=2),
    "no_bias": dict(bias=False),
    "integer_offsets": dict(channels_in=4, channels_out=3, dimensions=12, padding=1, _integer_offsets=True),
}


def make_deform1d_cases():
    ref = load_reference_test_module()
    out = {}
    names = []
    for idx, (name, kw) in enumerate(CASES_1D.items()):
        kw = dict(kw)
        torch.manual_seed(9876 + idx)
        integer = kw.pop("_integer_offsets", False)
        x, offset, alpha, weight, bias = ref.generate_data(1, device="cpu", dtype=torch.float64, **kw)
        if integer:
            offset = torch.randint(-2, 3, offset.shape).to(torch.float64)
        stride, padding, dilation = kw.get("stride", 1), kw.get("padding", 0), kw.get("dilation", 1)
        expected = ref.expected_fn(1, x, offset, alpha, weight, bias, stride, padding, dilation)
        names.append(name)
        out[f"{name}/x"] = x.numpy()
        out[f"{name}/offset"] = offset.numpy()
        out[f"{name}/mask"] = alpha.numpy()
        out[f"{name}/weight"] = weight.numpy()
        if bias is not None:
            out[f"{name}/bias"] = bias.numpy()
        out[f"{name}/expected"] = expected.numpy()
        out[f"{name}/geom"] = np.array([stride, padding, dilation, kw.get("n_weight_groups", 1),
                                        kw.get("n_offset_groups", 1)], dtype=np.int64)
        print(f"1d {name}: out {tuple(expected.shape)}", flush=True)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "deform1d_fwd_cases.npz"), **out)


if __name__ == "__main__":
    sets = sys.argv[2:] or ["size_map", "deform3d", "deform1d"]
    if "size_map" in sets:
        make_size_map_cases()
    if "deform3d" in sets:
        make_deform_cases()
    if "deform1d" in sets:
        make_deform1d_cases()
