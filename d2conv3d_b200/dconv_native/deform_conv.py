"""Functional and module front-ends with the call signatures of the reference's
ops/dconv-native/src/dconv_native/deform_conv.py (deform_conv3d :42-85,
DeformConvNd :88-151, DeformConv3d :175-209).  Note the reference's argument order:
the modulation mask `alpha` is the third positional argument.
"""
import math

import torch
from torch import nn
from torch.nn.modules.utils import _single, _triple

from . import _ops


def _upcast_if_any_half(tensors):
    """Reference behaviour (deform_conv.py:15-16,54-59): if any tensor is fp16, every
    tensor is converted to fp32 and the result stays fp32."""
    if any(t is not None and t.dtype == torch.half for t in tensors):
        return [None if t is None else t.float() for t in tensors]
    return list(tensors)


def deform_conv3d(input, offset, alpha, weight, bias=None, stride=(1, 1, 1), padding=(0, 0, 0),
                  dilation=(1, 1, 1), n_weight_groups=1, n_offset_groups=1):
    input, offset, alpha, weight, bias = _upcast_if_any_half((input, offset, alpha, weight, bias))
    s, p, d = _triple(stride), _triple(padding), _triple(dilation)
    return _ops.deform_conv3d(input, offset, alpha, weight, bias, s[0], s[1], s[2], p[0], p[1], p[2],
                              d[0], d[1], d[2], n_weight_groups, n_offset_groups)


def dyn_dilated_conv3d(input, size_map, alpha, weight, bias=None, mode="xyz", stride=(1, 1, 1),
                       padding=(0, 0, 0), dilation=(1, 1, 1), n_weight_groups=1, n_offset_groups=1):
    """deform_conv3d(input, offsets_from_size_map(size_map, mode, k, dilation) repeated per
    offset group, alpha, ...) evaluated without materialising the offsets; also returns the
    gradient w.r.t. size_map directly."""
    input, size_map, alpha, weight, bias = _upcast_if_any_half((input, size_map, alpha, weight, bias))
    return _ops.dyn_dilated_conv3d(input, size_map, alpha, weight, bias, mode.lower(), _triple(stride),
                                   _triple(padding), _triple(dilation), n_weight_groups, n_offset_groups)


def deform_conv1d(input, offset, alpha, weight, bias=None, stride=1, padding=0, dilation=1,
                  n_weight_groups=1, n_offset_groups=1):
    """ops/dconv-native/src/dconv_native/deform_conv.py:19-40: half inputs are up-cast; a missing bias or
    alpha stands for zeros / ones."""
    input, offset, alpha, weight, bias = _upcast_if_any_half((input, offset, alpha, weight, bias))
    return _ops.deform_conv1d(input, offset, alpha, weight, bias, stride, padding, dilation,
                              n_weight_groups, n_offset_groups)


class DeformConvNd(nn.Module):
    """Holds `weight` [Cout, Cin/groups, *k] and optional `bias` [Cout], initialised like
    nn.Conv3d (kaiming-uniform with a=sqrt(5); bias uniform in +-1/sqrt(fan_in))."""

    def __init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups,
                 offset_groups, bias):
        super().__init__()
        for value, by, msg in ((in_channels, groups, "in_channels must be divisible by groups"),
                               (in_channels, offset_groups, "in_channels must be divisible by offset_groups"),
                               (out_channels, groups, "out_channels must be divisible by groups")):
            if value % by != 0:
                raise ValueError(msg)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        self.groups, self.offset_groups = groups, offset_groups
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels // groups, *kernel_size))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = nn.init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in)
            nn.init.uniform_(self.bias, -bound, bound)

    def extra_repr(self):
        parts = [f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}"]
        if any(p != 0 for p in self.padding):
            parts.append(f"padding={self.padding}")
        if any(d != 1 for d in self.dilation):
            parts.append(f"dilation={self.dilation}")
        if self.groups != 1:
            parts.append(f"groups={self.groups}")
        if self.offset_groups != 1:
            parts.append(f"offset_groups={self.offset_groups}")
        if self.bias is None:
            parts.append("bias=False")
        return ", ".join(parts)


class DeformConv3d(DeformConvNd):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 offset_groups=1, bias=True):
        super().__init__(in_channels, out_channels, _triple(kernel_size), _triple(stride), _triple(padding),
                         _triple(dilation), groups, offset_groups, bias)

    def forward(self, input, offset, alpha):
        return deform_conv3d(input, offset, alpha, self.weight, self.bias, self.stride, self.padding,
                             self.dilation, self.groups, self.offset_groups)

    def forward_field(self, input, size_map, alpha, mode):
        """Same layer driven by a dilation field (see dyn_dilated_conv3d)."""
        return dyn_dilated_conv3d(input, size_map, alpha, self.weight, self.bias, mode, self.stride,
                                  self.padding, self.dilation, self.groups, self.offset_groups)


class DeformConv1d(DeformConvNd):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 offset_groups=1, bias=True):
        super().__init__(in_channels, out_channels, _single(kernel_size), _single(stride), _single(padding),
                         _single(dilation), groups, offset_groups, bias)

    def forward(self, input, offset, alpha):
        return deform_conv1d(input, offset, alpha, self.weight, self.bias, self.stride, self.padding,
                             self.dilation, self.groups, self.offset_groups)
