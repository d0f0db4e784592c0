"""CPU-only checks of the C ABI: the library loads, exports every symbol the header
declares, and its host-side validation / helper entry points behave (no kernel is
launched here)."""
import ctypes
import os
import re

import pytest

from d2conv3d_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from d2conv3d_b200 import build
    build.build()
    return _lib.lib()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "d2conv3d.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(d2c_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(L):
    names = _declared_symbols()
    assert len(names) >= 17
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/d2conv3d.h but not exported"


def _desc(**kw):
    base = dict(dtype=0, batch=2, in_channels=8, out_channels=8, in_d=4, in_h=6, in_w=6, kd=3, kh=3, kw=3,
                stride_d=1, stride_h=1, stride_w=1, pad_d=1, pad_h=1, pad_w=1, dil_d=1, dil_h=1, dil_w=1,
                groups=1, offset_groups=2)
    base.update(kw)
    return _lib.ConvDesc(**base)


def test_output_dims_formula(L):
    out = (ctypes.c_int32 * 3)()
    d = _desc(in_d=5, in_h=7, in_w=7, stride_h=2, pad_d=0, pad_h=1, pad_w=2, dil_w=2)
    assert L.d2c_output_dims(ctypes.byref(d), out) == 0
    assert tuple(out) == (3, 4, 7)   # the reference test's forward geometry
    d = _desc(in_d=1, pad_d=0)
    assert L.d2c_output_dims(ctypes.byref(d), out) == -5


def test_shape_checks(L):
    d = _desc()
    od = (ctypes.c_int64 * 4)(2 * 81, 4, 6, 6)
    md = (ctypes.c_int64 * 4)(2 * 27, 4, 6, 6)
    assert L.d2c_deform_conv3d_check(ctypes.byref(d), od, md) == 0
    assert L.d2c_deform_conv3d_check(ctypes.byref(d), od, None) == 0
    bad = (ctypes.c_int64 * 4)(81, 4, 6, 6)
    assert L.d2c_deform_conv3d_check(ctypes.byref(d), bad, md) == -6
    bad = (ctypes.c_int64 * 4)(2 * 27, 4, 6, 5)
    assert L.d2c_deform_conv3d_check(ctypes.byref(d), od, bad) == -7
    assert L.d2c_deform_conv3d_check(ctypes.byref(_desc(offset_groups=3)), od, md) == -4
    assert L.d2c_deform_conv3d_check(ctypes.byref(_desc(groups=3)), od, md) == -4
    assert L.d2c_deform_conv3d_check(ctypes.byref(_desc(stride_d=0)), od, md) == -3
    assert L.d2c_deform_conv3d_check(ctypes.byref(_desc(pad_w=-1)), od, md) == -3
    assert L.d2c_deform_conv3d_check(ctypes.byref(_desc(dtype=2)), od, md) == -2
    assert L.d2c_deform_conv3d_check(None, od, md) == -1


def test_null_pointers_rejected_before_any_launch(L):
    d = _desc()
    assert L.d2c_deform_conv3d_fwd(ctypes.byref(d), None, None, None, None, None, None, None, 0, None) == -1
    assert L.d2c_deform_conv3d_bwd(ctypes.byref(d), *([None] * 11), 0, None) == -1
    assert L.d2c_dyn_dilated_conv3d_fwd(ctypes.byref(d), 3, *([None] * 7), 0, None) == -1
    assert L.d2c_depthwise_conv3d_fwd(ctypes.byref(d), None, None, None, None, None) == -1


def test_status_strings(L):
    assert L.d2c_status_string(0) == b"ok"
    for code in list(range(-11, 0)) + [1, 2]:
        s = L.d2c_status_string(code)
        assert s and s != b"unknown status"
    assert L.d2c_status_string(99) == b"unknown status"


def test_math_mode_and_intermediate_cap(L):
    assert L.d2c_set_math_mode(7) == -10
    for name, code in _lib.MATH_MODES.items():
        _lib.set_math_mode(name)
        assert _lib.get_math_mode() == name
    _lib.set_math_mode("auto")
    from d2conv3d_b200.dconv_native import _ops
    default = _ops.config.get_max_intermediate_elements()
    assert default == 1 << 32   # reference default, csrc/ops/dconv3d_gpu.cu:12
    _ops.config.set_max_intermediate_elements(1000)
    assert _ops.config.get_max_intermediate_elements() == 1000
    # the cap bounds the backward's gradient-column scratch: one clip of 8*27*144 fp32 elements
    d = _desc()
    assert L.d2c_workspace_bytes(_lib.OP_DEFORM_BWD, ctypes.byref(d)) == 8 * 27 * 144 * 4
    _ops.config.set_max_intermediate_elements(default)
    assert L.d2c_workspace_bytes(_lib.OP_DEFORM_BWD, ctypes.byref(d)) == 2 * 8 * 27 * 144 * 4


def test_sample_cache_sizes_follow_mode_cap_and_shape(L):
    """d2c_sample_cache_bytes is pure host arithmetic: image (one 8 KB block per 64-channel slice and 64 voxels, hi and
    lo in the fp32-parity mode) + staged input + position records; 0 wherever the call pair would not use a cache."""
    mode0, cap0 = L.d2c_get_math_mode(), L.d2c_get_max_intermediate_elements()
    try:
        c2 = _desc(batch=2, in_channels=512, out_channels=512, in_d=8, in_h=30, in_w=54, offset_groups=8)
        V, tiles = 8 * 30 * 54, 2 * 102                      # 102 tiles of 128 voxels per clip
        pairs = 8 * 27 // 2                                  # 216 slices of 64 channels
        pos = 2 * 8 * 27 * V * 16
        L.d2c_set_math_mode(_lib.MATH_MODES["auto"])
        assert L.d2c_sample_cache_bytes(ctypes.byref(c2)) == tiles * 2 * pairs * 4 * 8192 + 2 * V * 512 * 4 + pos
        L.d2c_set_math_mode(_lib.MATH_MODES["bf16"])
        assert L.d2c_sample_cache_bytes(ctypes.byref(c2)) == tiles * 2 * pairs * 2 * 8192 + 2 * V * 512 * 2 + pos
        L.d2c_set_math_mode(_lib.MATH_MODES["fp32"])         # CUDA-core tier: nothing to keep
        assert L.d2c_sample_cache_bytes(ctypes.byref(c2)) == 0
        L.d2c_set_math_mode(_lib.MATH_MODES["auto"])
        L.d2c_set_max_intermediate_elements(2 * 512 * 27 * V - 1)      # one element under the image's size
        assert L.d2c_sample_cache_bytes(ctypes.byref(c2)) == 0
        L.d2c_set_max_intermediate_elements(cap0)
        assert L.d2c_sample_cache_bytes(ctypes.byref(_desc(dtype=1))) == 0          # float64
        assert L.d2c_sample_cache_bytes(ctypes.byref(_desc())) == 0                 # 4 channels per group: generic tier
        assert L.d2c_sample_cache_bytes(None) == 0
        assert L.d2c_bind_sample_cache(None) == 0                                   # unbinding is always allowed
    finally:
        L.d2c_set_math_mode(mode0)
        L.d2c_set_max_intermediate_elements(cap0)
