"""The C++ route of the drop-in: the reference's own pybind module and autograd nodes (csrc/ops/dconv.cpp,
dconv3d.h:70-226, dconv1d.h:69-186, compiled unmodified) running on libd2conv3d.so through
baseline/binding/d2c_dconv_binding.cpp, which replaces nothing but the reference's two .cu files.  Built by
baseline/build_binding.py into baseline/_ref/_binding (skipped when that build is absent).

Checked: same results as this repository's Python route (which calls the same C ABI) and as the reference's own
compiled extension, forward and every gradient, fp64 and fp32, with and without mask / bias; the 1-D op; the
`config` sub-module."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from tests import _reference
from tests._util import make_problem

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO = os.path.join(ROOT, "baseline", "_ref", "_binding", "dconv_d2c_ops.so")


@pytest.fixture(scope="module")
def binding():
    if not os.path.exists(SO):
        pytest.skip("baseline/_ref/_binding/dconv_d2c_ops.so not built (baseline/build_binding.py)")
    from d2conv3d_b200 import _lib
    _lib.lib()                                   # the same libd2conv3d.so the binding links against
    spec = importlib.util.spec_from_file_location("dconv_d2c_ops", SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run(fn, tensors, gy, *geom):
    ts = [None if t is None else t.detach().clone().requires_grad_() for t in tensors]
    y = fn(*ts, *geom)
    y.backward(gy)
    torch.cuda.synchronize()
    return [y.detach()] + [None if t is None else t.grad for t in ts]


CASES = [
    dict(dtype=np.float64, B=2, Cin=6, Cout=4, dims=(4, 5, 6), G=2, padding=1, mask=True, bias=True),
    dict(dtype=np.float64, B=1, Cin=4, Cout=6, dims=(3, 6, 5), G=1, padding=(0, 1, 2), stride=(1, 2, 1), dilation=(1, 1, 2),
         groups=2, mask=False, bias=False),
    dict(dtype=np.float32, B=2, Cin=128, Cout=64, dims=(3, 8, 9), G=2, padding=1, mask=True, bias=True),   # tensor-core tier
]


@pytest.mark.parametrize("ci", range(len(CASES)))
def test_reference_autograd_node_on_this_library_matches_python_route_and_reference(binding, ci):
    from d2conv3d_b200 import dconv_native
    cfg = dict(CASES[ci])
    dtype, has_mask, has_bias = cfg.pop("dtype"), cfg.pop("mask"), cfg.pop("bias")
    p = make_problem(500 + ci, dtype=dtype, offset_std=1.5, mask=has_mask, bias=has_bias, **cfg)
    cu = lambda a: None if a is None else torch.from_numpy(a).cuda()
    tensors = [cu(p[k]) for k in ("x", "geo", "mask", "weight", "bias")]
    gy = cu(p["gy"])
    geom = (*p["stride"], *p["padding"], *p["dilation"], p["groups"], p["offset_groups"])
    got = run(binding.deform_conv3d, tensors, gy, *geom)
    ours = run(dconv_native._ops.deform_conv3d, tensors, gy, *geom)
    tol = 1e-12 if dtype == np.float64 else 1e-5          # same kernels: only atomic summation order may differ
    for a, b in zip(got, ours):
        assert (a is None) == (b is None)
        if a is not None:
            assert float((a - b).abs().max()) <= tol * max(float(b.abs().max()), 1e-30)
    ref = _reference.load("dconv_native")
    if ref is not None:
        want = run(ref._ops.deform_conv3d, tensors, gy, *geom)
        tol = 1e-10 if dtype == np.float64 else 1e-4
        for name, a, b in zip(("y", "gx", "goff", "gmask", "gw", "gbias"), got, want):
            if b is not None and b.defined() if hasattr(b, "defined") else b is not None:
                assert float((a - b).abs().max()) <= tol * max(float(b.abs().max()), 1e-30), name


def test_reference_conv1d_node_on_this_library(binding):
    from d2conv3d_b200 import dconv_native
    g = torch.Generator().manual_seed(77)
    B, C, Cout, L, K, G = 2, 8, 6, 21, 3, 2
    x = torch.randn(B, C, L, generator=g, dtype=torch.float64).cuda()
    off = (torch.randn(B, G * K, L, generator=g, dtype=torch.float64) * 1.5).cuda()
    off.view(-1)[::4] = torch.round(off.view(-1)[::4])          # some exactly-integer positions
    alpha = torch.sigmoid(torch.randn(B, G * K, L, generator=g, dtype=torch.float64)).cuda()
    w = torch.randn(Cout, C, K, generator=g, dtype=torch.float64).cuda()
    b = torch.randn(Cout, generator=g, dtype=torch.float64).cuda()
    gy = torch.randn(B, Cout, L, generator=g, dtype=torch.float64).cuda()
    got = run(binding.deform_conv1d, [x, off, alpha, w, b], gy, 1, 1, 1, 1, G)
    ours = run(dconv_native._ops.deform_conv1d, [x, off, alpha, w, b], gy, 1, 1, 1, 1, G)
    for a, c in zip(got, ours):
        assert float((a - c).abs().max()) <= 1e-12 * float(c.abs().max())
    ref = _reference.load("dconv_native")
    if ref is not None:
        want = run(ref._ops.deform_conv1d, [x, off, alpha, w, b], gy, 1, 1, 1, 1, G)
        for a, c in zip(got, want):
            assert float((a - c).abs().max()) <= 1e-10 * float(c.abs().max())


def test_config_submodule_and_error_conversion(binding):
    old = binding.config.get_max_intermediate_elements()
    binding.config.set_max_intermediate_elements(12345)
    assert binding.config.get_max_intermediate_elements() == 12345
    binding.config.set_max_intermediate_elements(old)
    x = torch.randn(1, 4, 3, 4, 4, device="cuda")
    w = torch.randn(4, 4, 3, 3, 3, device="cuda")
    bad_offset = torch.zeros(1, 80, 1, 2, 2, device="cuda")    # 81 channels expected
    with pytest.raises(RuntimeError):
        binding.deform_conv3d(x, bad_offset, None, w, None, 1, 1, 1, 0, 0, 0, 1, 1, 1, 1, 1)
