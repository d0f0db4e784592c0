"""Seeded random sweep of the tensor-core tier against the oracle: random clip counts, volume sizes, kernel
shapes, strides, paddings, dilations, offset groups, channel counts (multiples of 64, Cout up to 512), with and
without mask / bias, offset spreads from 0 (integer coordinates) to 3 voxels -- forward and all gradients, in
the fp32-parity mode (1e-4 of scale) and in the single-pass bf16 mode (its stated 1e-2 / 2e-2)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests._util import make_problem

pytestmark = pytest.mark.gpu

BOUNDS = {"auto": (1e-4, 1e-4), "bf16": (1e-2, 2e-2)}


def random_case(i):
    rng = np.random.default_rng(9000 + i)
    k = tuple(int(v) for v in rng.choice([1, 3], size=3))
    if k == (1, 1, 1) and i % 2:
        k = (3, 3, 3)
    dil = tuple(int(v) for v in rng.choice([1, 2], size=3))
    stride = tuple(int(v) for v in rng.choice([1, 1, 2], size=3))
    pad = tuple(int(rng.integers(0, d * (kk // 2) + 1)) for d, kk in zip(dil, k))
    dims = tuple(int(rng.integers(max(2, d * (kk - 1) + 1 - 2 * p), 11)) for d, kk, p in zip(dil, k, pad))
    G = int(rng.choice([1, 2]))
    Cin = 64 * G * int(rng.choice([1, 2]))
    Cout = 64 * int(rng.choice([1, 2, 3, 5, 8]))
    return dict(B=int(rng.integers(1, 4)), Cin=Cin, Cout=Cout, dims=dims, k=k, stride=stride, padding=pad,
                dilation=dil, G=G, mask=bool(rng.integers(0, 2)), bias=bool(rng.integers(0, 2)),
                offset_std=float(rng.choice([0.0, 0.5, 1.5, 3.0])))


@pytest.mark.parametrize("mode", ["auto", "bf16"])
@pytest.mark.parametrize("i", range(16))
def test_random_geometry_vs_oracle(mode, i):
    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native
    cfg = random_case(i)
    p = make_problem(9100 + i, dtype=np.float32, **cfg)
    if cfg["offset_std"] == 0.0:      # integer sampling positions, some of them exactly on / beyond the border
        p["geo"][:] = np.random.default_rng(i).integers(-3, 4, size=p["geo"].shape).astype(np.float32)
    kw = dict(stride=p["stride"], padding=p["padding"], dilation=p["dilation"], groups=1, offset_groups=cfg["G"])
    d = lambda a: None if a is None else a.astype(np.float64)
    want_y = orc.deform_conv3d_fwd(d(p["x"]), d(p["geo"]), d(p["mask"]), d(p["weight"]), d(p["bias"]), **kw)
    want_g = orc.deform_conv3d_bwd(d(p["gy"]), d(p["x"]), d(p["geo"]), d(p["mask"]), d(p["weight"]),
                                   p["bias"] is not None, **kw)
    d2conv3d_b200.set_math_mode(mode)
    try:
        names = ("x", "geo", "mask", "weight", "bias")
        ts = [None if p[n] is None else torch.from_numpy(p[n]).cuda().requires_grad_() for n in names]
        _lib.profile_read(); _lib.profile_enable(True)
        y = dconv_native.deform_conv3d(*ts, p["stride"], p["padding"], p["dilation"], 1, cfg["G"])
        y.backward(torch.from_numpy(p["gy"]).cuda())
        _lib.profile_enable(False)
        phases = [n for n, _ in _lib.profile_read()]
        assert "fwd_sm100_fused" in phases and "bwd_dcol_sm100" in phases, (cfg, phases)
        _lib.device_status()
    finally:
        d2conv3d_b200.set_math_mode("auto")
    fb, gb = BOUNDS[mode]
    scale = max(np.abs(want_y).max(), 1e-30)
    assert np.abs(y.detach().cpu().numpy() - want_y).max() <= fb * scale, cfg
    for t, w_, n in zip(ts, want_g, names):
        if t is None:
            continue
        gs = np.abs(w_).max()
        if gs == 0:
            assert float(t.grad.abs().max()) == 0.0, (cfg, n)
        else:
            assert np.abs(t.grad.cpu().numpy() - w_).max() <= gb * gs, (cfg, n)
