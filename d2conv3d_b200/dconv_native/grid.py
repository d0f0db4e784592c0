"""Dilation field -> offsets, with the semantics of the reference's
`offsets_from_size_map` (utils/grid.py:72-98; the older copy shipped inside the
extension, ops/dconv-native/src/dconv_native/grid.py:62-80, infers the mode from the
channel count).  Plain PyTorch: this is the materialising route; the fused route is
`dyn_dilated_conv3d`, which never builds the 3*K offset channels.
"""
import torch
from torch.nn.modules.utils import _triple

_MODE_BY_CHANNELS = {1: "x", 2: "xy", 3: "xyz"}


def get_kernel_grid(kernel_shape, dilation, device="cpu", dtype=None):
    """[3, kd, kh, kw]: per-dim tap positions linspace(-dil*(k//2), dil*(k//2), k)."""
    axes = [torch.linspace(-d * (k // 2), d * (k // 2), k, device=device, dtype=dtype)
            for d, k in zip(dilation, kernel_shape)]
    return torch.stack(torch.meshgrid(axes, indexing="ij"))


def expand_size_map(size_map, mode):
    """[B, n, D, H, W] -> [B, 3, D, H, W] in (z, y, x) order; absent dims are ones."""
    n = size_map.shape[1]
    ones = torch.ones_like(size_map[:, :1])
    if mode == "xyz":
        want, parts = 3, None
    elif mode == "xxz":
        want, parts = 2, (size_map[:, 0:1], size_map[:, 1:2], size_map[:, 1:2])
    elif mode == "xy":
        want, parts = 2, (ones, size_map[:, 0:1], size_map[:, 1:2])
    elif mode == "x":
        want, parts = 1, (ones, size_map, size_map)
    else:
        raise ValueError(f"Unknown offset mode '{mode}'")
    if n != want:
        raise ValueError(f"mode '{mode}' needs a size_map with {want} channels, got {n}")
    return size_map if parts is None else torch.cat(parts, dim=1)


def offsets_from_size_map(size_map, *args, **kwargs):
    """offsets[b, (tap, zyx), d, h, w] = kernel_grid[zyx, tap] * (size[b, zyx, d, h, w] - 1).

    Accepts both reference signatures:
      offsets_from_size_map(size_map, mode, kernel_shape=(3,3,3), dilation=(1,1,1))
      offsets_from_size_map(size_map, kernel_shape=(3,3,3), dilation=(1,1,1))   # mode from channels
    """
    args = list(args)
    mode = kwargs.pop("mode", None)
    if args and isinstance(args[0], str):
        mode = args.pop(0)
    kernel_shape = kwargs.pop("kernel_shape", args.pop(0) if args else (3, 3, 3))
    dilation = kwargs.pop("dilation", args.pop(0) if args else (1, 1, 1))
    if kwargs or args:
        raise TypeError("unexpected arguments")
    if mode is None:
        if size_map.shape[1] not in _MODE_BY_CHANNELS:
            raise ValueError(f"size_map should have 1, 2, or 3 channels, but has {size_map.shape[1]}")
        mode = _MODE_BY_CHANNELS[size_map.shape[1]]
    kernel_shape, dilation = _triple(kernel_shape), _triple(dilation)
    base = get_kernel_grid(kernel_shape, dilation, size_map.device)            # [3, kd, kh, kw] fp32
    K = kernel_shape[0] * kernel_shape[1] * kernel_shape[2]
    base = base.reshape(3, K).t().reshape(1, K, 3, 1, 1, 1)                     # [1, K, zyx, 1,1,1]
    size3 = expand_size_map(size_map, mode.lower()).unsqueeze(1)               # [B, 1, zyx, D,H,W]
    offsets = base * (size3 - 1)
    B, _, _, D, H, W = offsets.shape
    return offsets.reshape(B, K * 3, D, H, W)
