"""TEST INFRASTRUCTURE -- numpy front-end of the CPU oracle (liboracle built from
d2c_oracle.c).  Only tests, the smoke check and the bench's CPU-baseline legs
import this module; the product package never does.

All functions take / return C-contiguous numpy arrays (float32 or float64, one
dtype per call) in the reference's NCDHW conventions.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libd2c_oracle.so")

FIELD_MODES = {"x": 0, "xy": 1, "xxz": 2, "xyz": 3}
FIELD_CHANNELS = {"x": 1, "xy": 2, "xxz": 2, "xyz": 3}


class ConvDesc(ctypes.Structure):
    """Mirror of d2c_conv_desc (include/d2conv3d.h)."""

    _fields_ = [(n, ctypes.c_int32) for n in (
        "dtype", "batch", "in_channels", "out_channels", "in_d", "in_h", "in_w",
        "kd", "kh", "kw", "stride_d", "stride_h", "stride_w", "pad_d", "pad_h", "pad_w",
        "dil_d", "dil_h", "dil_w", "groups", "offset_groups")]


def build(force=False):
    """Compile the oracle with the Makefile next to this file."""
    srcs = [os.path.join(_HERE, f) for f in ("d2c_oracle.c", "d2c_oracle_impl.inc", "Makefile")]
    if (not force and os.path.exists(_LIB_PATH)
            and all(os.path.getmtime(_LIB_PATH) >= os.path.getmtime(s) for s in srcs)):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def set_threads(n=0):
    """Sets the OpenMP team size of the oracle's loops (n <= 0: leave it) and returns the size in effect."""
    f = lib().orc_set_threads
    f.argtypes, f.restype = [ctypes.c_int], ctypes.c_int
    return int(f(int(n)))


def _triple(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v, v)


def make_desc(x_shape, w_shape, stride=1, padding=0, dilation=1, groups=1, offset_groups=1,
              dtype=np.float32):
    s, p, d = _triple(stride), _triple(padding), _triple(dilation)
    B, Cin, D, H, W = x_shape
    return ConvDesc(0 if np.dtype(dtype) == np.float32 else 1, B, Cin, w_shape[0], D, H, W,
                    w_shape[2], w_shape[3], w_shape[4], s[0], s[1], s[2], p[0], p[1], p[2],
                    d[0], d[1], d[2], groups, offset_groups)


def output_dims(desc):
    out = (ctypes.c_int32 * 3)()
    if lib().orc_output_dims(ctypes.byref(desc), out):
        raise ValueError("bad geometry")
    return tuple(out)


def _suffix(dtype):
    return "_f32" if np.dtype(dtype) == np.float32 else "_f64"


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def _fn(name, dtype):
    f = getattr(lib(), name + _suffix(dtype))
    f.restype = ctypes.c_int
    return f


def deform_conv3d_fwd(x, offset, mask, w, bias=None, stride=1, padding=0, dilation=1, groups=1,
                      offset_groups=1):
    dt = x.dtype
    x, offset, mask, w, bias = (_c(a, dt) for a in (x, offset, mask, w, bias))
    desc = make_desc(x.shape, w.shape, stride, padding, dilation, groups, offset_groups, dt)
    y = np.empty((x.shape[0], w.shape[0]) + output_dims(desc), dtype=dt)
    rc = _fn("orc_deform_conv3d_fwd", dt)(ctypes.byref(desc), _p(x), _p(offset), _p(mask), _p(w),
                                          _p(bias), _p(y))
    if rc:
        raise RuntimeError(f"oracle fwd failed: {rc}")
    return y


def deform_conv3d_bwd(gy, x, offset, mask, w, has_bias=True, stride=1, padding=0, dilation=1,
                      groups=1, offset_groups=1):
    """Returns (grad_x, grad_offset, grad_mask or None, grad_w, grad_bias or None)."""
    dt = x.dtype
    gy, x, offset, mask, w = (_c(a, dt) for a in (gy, x, offset, mask, w))
    desc = make_desc(x.shape, w.shape, stride, padding, dilation, groups, offset_groups, dt)
    gx, goff, gw = np.empty_like(x), np.empty_like(offset), np.empty_like(w)
    gmask = np.empty_like(mask) if mask is not None else None
    gb = np.empty((w.shape[0],), dtype=dt) if has_bias else None
    rc = _fn("orc_deform_conv3d_bwd", dt)(ctypes.byref(desc), _p(gy), _p(x), _p(offset), _p(mask),
                                          _p(w), _p(gx), _p(goff), _p(gmask), _p(gw), _p(gb))
    if rc:
        raise RuntimeError(f"oracle bwd failed: {rc}")
    return gx, goff, gmask, gw, gb


def deform_conv3d_corners(x_shape, w_shape, offset, stride=1, padding=0, dilation=1,
                          offset_groups=1):
    dt = offset.dtype
    offset = _c(offset, dt)
    desc = make_desc(x_shape, w_shape, stride, padding, dilation, 1, offset_groups, dt)
    K = w_shape[2] * w_shape[3] * w_shape[4]
    V = int(np.prod(output_dims(desc)))
    out = np.empty((x_shape[0], offset_groups * K, 3, V), dtype=np.int32)
    getattr(lib(), "orc_deform_conv3d_corners" + _suffix(dt))(ctypes.byref(desc), _p(offset), _p(out))
    return out


def offsets_from_size_map(size_map, mode, kernel_shape=(3, 3, 3), dilation=(1, 1, 1)):
    """[B, n, D, H, W] -> [B, 3K, D, H, W]; spatial dims are OUTPUT dims."""
    dt = size_map.dtype
    size_map = _c(size_map, dt)
    B, _, D, H, W = size_map.shape
    k, dil = _triple(kernel_shape), _triple(dilation)
    # geometry whose output dims equal the field's dims ("same" conv of stride 1)
    pad = tuple(dd * (kk - 1) // 2 for kk, dd in zip(k, dil))
    ext = tuple(dd * (kk - 1) - 2 * pp for kk, dd, pp in zip(k, dil, pad))
    desc = make_desc((B, 1, D + ext[0], H + ext[1], W + ext[2]), (1, 1) + k, 1, pad, dil, 1, 1, dt)
    assert output_dims(desc) == (D, H, W)
    out = np.empty((B, 3 * k[0] * k[1] * k[2], D, H, W), dtype=dt)
    getattr(lib(), "orc_offsets_from_size_map" + _suffix(dt))(
        ctypes.byref(desc), FIELD_MODES[mode], _p(size_map), _p(out))
    return out


def dyn_dilated_conv3d_fwd(x, size_map, mask, w, bias=None, mode="xyz", stride=1, padding=0,
                           dilation=1, groups=1, offset_groups=1):
    dt = x.dtype
    x, size_map, mask, w, bias = (_c(a, dt) for a in (x, size_map, mask, w, bias))
    desc = make_desc(x.shape, w.shape, stride, padding, dilation, groups, offset_groups, dt)
    y = np.empty((x.shape[0], w.shape[0]) + output_dims(desc), dtype=dt)
    rc = _fn("orc_dyn_dilated_conv3d_fwd", dt)(ctypes.byref(desc), FIELD_MODES[mode], _p(x),
                                               _p(size_map), _p(mask), _p(w), _p(bias), _p(y))
    if rc:
        raise RuntimeError(f"oracle dyn fwd failed: {rc}")
    return y


def dyn_dilated_conv3d_bwd(gy, x, size_map, mask, w, has_bias=True, mode="xyz", stride=1,
                           padding=0, dilation=1, groups=1, offset_groups=1):
    dt = x.dtype
    gy, x, size_map, mask, w = (_c(a, dt) for a in (gy, x, size_map, mask, w))
    desc = make_desc(x.shape, w.shape, stride, padding, dilation, groups, offset_groups, dt)
    gx, gs, gw = np.empty_like(x), np.empty_like(size_map), np.empty_like(w)
    gmask = np.empty_like(mask) if mask is not None else None
    gb = np.empty((w.shape[0],), dtype=dt) if has_bias else None
    rc = _fn("orc_dyn_dilated_conv3d_bwd", dt)(
        ctypes.byref(desc), FIELD_MODES[mode], _p(gy), _p(x), _p(size_map), _p(mask), _p(w),
        _p(gx), _p(gs), _p(gmask), _p(gw), _p(gb))
    if rc:
        raise RuntimeError(f"oracle dyn bwd failed: {rc}")
    return gx, gs, gmask, gw, gb


def dyn_dilated_conv3d_corners(x_shape, w_shape, size_map, mode, stride=1, padding=0, dilation=1,
                               offset_groups=1):
    dt = size_map.dtype
    size_map = _c(size_map, dt)
    desc = make_desc(x_shape, w_shape, stride, padding, dilation, 1, offset_groups, dt)
    K = w_shape[2] * w_shape[3] * w_shape[4]
    V = int(np.prod(output_dims(desc)))
    out = np.empty((x_shape[0], offset_groups * K, 3, V), dtype=np.int32)
    getattr(lib(), "orc_dyn_dilated_conv3d_corners" + _suffix(dt))(
        ctypes.byref(desc), FIELD_MODES[mode], _p(size_map), _p(out))
    return out


def depthwise_conv3d_fwd(x, w, bias=None, stride=1, padding=0, dilation=1):
    dt = x.dtype
    x, w, bias = (_c(a, dt) for a in (x, w, bias))
    desc = make_desc(x.shape, w.shape, stride, padding, dilation, x.shape[1], 1, dt)
    y = np.empty((x.shape[0], w.shape[0]) + output_dims(desc), dtype=dt)
    rc = _fn("orc_depthwise_conv3d_fwd", dt)(ctypes.byref(desc), _p(x), _p(w), _p(bias), _p(y))
    if rc:
        raise RuntimeError(f"oracle depthwise fwd failed: {rc}")
    return y


def depthwise_conv3d_bwd(gy, x, w, has_bias=True, stride=1, padding=0, dilation=1):
    dt = x.dtype
    gy, x, w = (_c(a, dt) for a in (gy, x, w))
    desc = make_desc(x.shape, w.shape, stride, padding, dilation, x.shape[1], 1, dt)
    gx, gw = np.empty_like(x), np.empty_like(w)
    gb = np.empty((w.shape[0],), dtype=dt) if has_bias else None
    rc = _fn("orc_depthwise_conv3d_bwd", dt)(ctypes.byref(desc), _p(gy), _p(x), _p(w), _p(gx),
                                             _p(gw), _p(gb))
    if rc:
        raise RuntimeError(f"oracle depthwise bwd failed: {rc}")
    return gx, gw, gb


def deform_conv1d_fwd(x, offset, alpha, weight, bias=None, stride=1, padding=0, dilation=1, groups=1,
                      offset_groups=1):
    """Modulated deformable conv1d, restating ops/dconv-native/csrc/ops/dconv1d_gpu.cu:24-55 (im2col with
    `a * lerp(v0, v1, x - x0)`, neighbours outside [0, L) read as 0) followed by the grouped GEMM + bias of
    :95-160.  numpy, small cases only.  x [B, C, L], offset / alpha [B, G*K, Lo], weight [Cout, C/groups, K]."""
    x = np.asarray(x); offset = np.asarray(offset); weight = np.asarray(weight)
    B, C, L = x.shape
    Cout, Cg, K = weight.shape
    Lo = (L + 2 * padding - dilation * (K - 1) - 1) // stride + 1
    assert offset.shape == (B, offset_groups * K, Lo)
    if alpha is None:
        alpha = np.ones_like(offset)
    cpg = C // offset_groups
    cols = np.zeros((B, C, K, Lo), dtype=x.dtype)
    ox = np.arange(Lo)
    for g in range(offset_groups):
        for i in range(K):
            pos = (ox * stride - padding + i * dilation).astype(x.dtype)[None, :] + offset[:, g * K + i, :]   # [B, Lo]
            x0 = np.floor(pos).astype(np.int64)
            x1 = x0 + 1
            t = pos - x0.astype(x.dtype)
            a = alpha[:, g * K + i, :]
            for c in range(g * cpg, (g + 1) * cpg):
                xc = x[:, c, :]                                           # [B, L]
                v0 = np.where((x0 >= 0) & (x0 < L), np.take_along_axis(xc, np.clip(x0, 0, L - 1), axis=1), 0)
                v1 = np.where((x1 >= 0) & (x1 < L), np.take_along_axis(xc, np.clip(x1, 0, L - 1), axis=1), 0)
                cols[:, c, i, :] = a * (v0 + t * (v1 - v0))
    y = np.zeros((B, Cout, Lo), dtype=x.dtype)
    cog = Cout // groups
    for gw in range(groups):
        wg = weight[gw * cog:(gw + 1) * cog].reshape(cog, Cg * K)
        cg = cols[:, gw * Cg:(gw + 1) * Cg].reshape(B, Cg * K, Lo)
        y[:, gw * cog:(gw + 1) * cog] = np.einsum("ok,bkl->bol", wg, cg)
    if bias is not None:
        y += np.asarray(bias)[None, :, None]
    return y


def _cols_1d(x, offset, alpha, K, stride, padding, dilation, offset_groups):
    """im2col of the 1-D op (dconv1d_gpu.cu:36-54): cols[b, c, i, ox] = a * lerp(v0, v1, x - x0)."""
    B, C, L = x.shape
    Lo = offset.shape[2]
    cpg = C // offset_groups
    cols = np.zeros((B, C, K, Lo), dtype=x.dtype)
    ox = np.arange(Lo)
    for g in range(offset_groups):
        for i in range(K):
            pos = (ox * stride - padding + i * dilation).astype(x.dtype)[None, :] + offset[:, g * K + i, :]   # [B, Lo]
            x0 = np.floor(pos).astype(np.int64)
            x1 = x0 + 1
            t = pos - x0.astype(x.dtype)
            a = alpha[:, g * K + i, :]
            for c in range(g * cpg, (g + 1) * cpg):
                xc = x[:, c, :]                                           # [B, L]
                v0 = np.where((x0 >= 0) & (x0 < L), np.take_along_axis(xc, np.clip(x0, 0, L - 1), axis=1), 0)
                v1 = np.where((x1 >= 0) & (x1 < L), np.take_along_axis(xc, np.clip(x1, 0, L - 1), axis=1), 0)
                cols[:, c, i, :] = a * (v0 + t * (v1 - v0))
    return cols


def deform_conv1d_bwd(gy, x, offset, alpha, weight, has_bias=True, stride=1, padding=0, dilation=1, groups=1,
                      offset_groups=1):
    """All five gradients of the modulated deformable conv1d, restating
    ops/dconv-native/csrc/ops/dconv1d_gpu.cu: gradient columns (:459-480), grad_input scatter with the
    `x1 - x < 1` test (:200-240), grad_offset / grad_alpha with the integer-position rule `x0 -= 1` when
    x - x0 < 1e-8 (:300-349), grad_weight from the re-computed columns (:499-536), grad_bias (:537).
    numpy, small cases only.  Returns (grad_x, grad_offset, grad_alpha, grad_weight, grad_bias or None)."""
    gy = np.asarray(gy); x = np.asarray(x); offset = np.asarray(offset); weight = np.asarray(weight)
    B, C, L = x.shape
    Cout, Cg, K = weight.shape
    Lo = gy.shape[2]
    had_alpha = alpha is not None
    alpha = np.ones_like(offset) if alpha is None else np.asarray(alpha)
    cog = Cout // groups
    cpg = C // offset_groups
    dcol = np.zeros((B, C, K, Lo), dtype=x.dtype)
    for gw in range(groups):
        wg = weight[gw * cog:(gw + 1) * cog]                                        # [cog, Cg, K]
        dcol[:, gw * Cg:(gw + 1) * Cg] = np.einsum("bol,ock->bckl", gy[:, gw * cog:(gw + 1) * cog], wg)
    gx = np.zeros_like(x)
    goff = np.zeros_like(offset)
    galpha = np.zeros_like(offset)
    ox = np.arange(Lo)
    bi = np.arange(B)[:, None]
    for g in range(offset_groups):
        for i in range(K):
            pos = (ox * stride - padding + i * dilation).astype(x.dtype)[None, :] + offset[:, g * K + i, :]
            a = alpha[:, g * K + i, :]
            x0 = np.floor(pos).astype(np.int64)
            x1 = x0 + 1
            # scatter (:221-236)
            w0 = 1 - (pos - x0)
            w1 = pos - x0
            ok0 = (x0 >= 0) & (x0 < L)
            ok1 = (x1 >= 0) & (x1 < L) & ((x1 - pos) < 1)
            # coordinate gradient (:329-346)
            x0g = np.where((pos - x0) < 1e-8, x0 - 1, x0)
            tg = pos - x0g
            for c in range(g * cpg, (g + 1) * cpg):
                col = dcol[:, c, i, :]
                grad = a * col
                np.add.at(gx[:, c, :], (np.broadcast_to(bi, x0.shape)[ok0], x0[ok0]), (w0 * grad)[ok0])
                np.add.at(gx[:, c, :], (np.broadcast_to(bi, x1.shape)[ok1], x1[ok1]), (w1 * grad)[ok1])
                xc = x[:, c, :]
                v0 = np.where((x0g >= 0) & (x0g < L), np.take_along_axis(xc, np.clip(x0g, 0, L - 1), axis=1), 0)
                v1 = np.where((x1 >= 0) & (x1 < L), np.take_along_axis(xc, np.clip(x1, 0, L - 1), axis=1), 0)
                galpha[:, g * K + i, :] += col * (tg * v1 + (-tg * v0 + v0))
                goff[:, g * K + i, :] += (v1 - v0) * col * a
    cols = _cols_1d(x, offset, alpha, K, stride, padding, dilation, offset_groups)
    gwt = np.zeros_like(weight)
    for gw in range(groups):
        gwt[gw * cog:(gw + 1) * cog] = np.einsum("bol,bckl->ock", gy[:, gw * cog:(gw + 1) * cog],
                                                 cols[:, gw * Cg:(gw + 1) * Cg])
    gb = gy.sum(axis=(0, 2)) if has_bias else None
    return gx, goff, (galpha if had_alpha else None), gwt, gb
