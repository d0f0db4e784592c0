"""Shared helpers of the test-suite: golden-case loading and seeded problem generation."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

_deform = None
_size = None


def deform_cases():
    global _deform
    if _deform is None:
        _deform = np.load(os.path.join(GOLDEN, "deform_fwd_cases.npz"))
    return _deform


def deform_case_names():
    return [str(n) for n in deform_cases()["names"]]


def load_deform_case(name, dtype=np.float64):
    d = deform_cases()
    g = [int(v) for v in d[f"{name}/geom"]]
    bias = d[f"{name}/bias"].astype(dtype) if f"{name}/bias" in d else None
    return dict(
        x=d[f"{name}/x"].astype(dtype), offset=d[f"{name}/offset"].astype(dtype),
        mask=d[f"{name}/mask"].astype(dtype), weight=d[f"{name}/weight"].astype(dtype), bias=bias,
        expected=d[f"{name}/expected"], stride=tuple(g[0:3]), padding=tuple(g[3:6]), dilation=tuple(g[6:9]),
        groups=g[9], offset_groups=g[10])


def size_map_cases():
    global _size
    if _size is None:
        _size = np.load(os.path.join(GOLDEN, "size_map_cases.npz"))
    return _size


def out_dims(in_dims, k, s, p, d):
    return tuple((i + 2 * pp - (dd * (kk - 1) + 1)) // ss + 1 for i, kk, ss, pp, dd in zip(in_dims, k, s, p, d))


def t3(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v, v)


def make_problem(seed, B, Cin, Cout, dims, k=3, stride=1, padding=0, dilation=1, groups=1, G=1, dtype=np.float32,
                 offset_std=1.0, bias=True, mask=True, field_mode=None):
    """Seeded synthetic problem in the style of the benchmark configurations: x ~ N(0,1), offsets ~ N(0, offset_std),
    mask = sigmoid(N(0,1)), weight ~ Kaiming-normal, bias ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    k, s, p, d = t3(k), t3(stride), t3(padding), t3(dilation)
    od = out_dims(dims, k, s, p, d)
    K = k[0] * k[1] * k[2]
    x = rng.standard_normal((B, Cin) + tuple(dims))
    if field_mode is None:
        geo = rng.standard_normal((B, G * 3 * K) + od) * offset_std
    else:
        nch = {"x": 1, "xy": 2, "xxz": 2, "xyz": 3}[field_mode]
        geo = 1 + np.log1p(np.exp(rng.standard_normal((B, nch) + od)))   # 1 + softplus(N(0,1))
    m = 1 / (1 + np.exp(-rng.standard_normal((B, G * K) + od))) if mask else None
    fan_in = (Cin // groups) * K
    w = rng.standard_normal((Cout, Cin // groups) + k) * np.sqrt(2.0 / fan_in)
    b = rng.standard_normal((Cout,)) if bias else None
    gy = rng.standard_normal((B, Cout) + od)
    cast = lambda a: None if a is None else np.ascontiguousarray(a, dtype=dtype)
    return dict(x=cast(x), geo=cast(geo), mask=cast(m), weight=cast(w), bias=cast(b), gy=cast(gy),
                stride=s, padding=p, dilation=d, groups=groups, offset_groups=G, out_dims=od)


_deform1d = None


def deform1d_cases():
    global _deform1d
    if _deform1d is None:
        _deform1d = np.load(os.path.join(GOLDEN, "deform1d_fwd_cases.npz"))
    return _deform1d


def deform1d_case_names():
    return [str(n) for n in deform1d_cases()["names"]]


def load_deform1d_case(name, dtype=np.float64):
    d = deform1d_cases()
    g = [int(v) for v in d[f"{name}/geom"]]
    bias = d[f"{name}/bias"].astype(dtype) if f"{name}/bias" in d else None
    return dict(x=d[f"{name}/x"].astype(dtype), offset=d[f"{name}/offset"].astype(dtype),
                mask=d[f"{name}/mask"].astype(dtype), weight=d[f"{name}/weight"].astype(dtype), bias=bias,
                expected=d[f"{name}/expected"], stride=g[0], padding=g[1], dilation=g[2], groups=g[3],
                offset_groups=g[4])
