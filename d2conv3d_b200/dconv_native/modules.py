"""Packaged deformable layers: a predictor conv (`deform_params`) produces offsets /
modulation mask / dilation field from the layer input, and `deform_conv`
(DeformConv3d) consumes them.

Class names, constructor arguments, sub-module names (`deform_params`,
`deform_conv`) and initialisation follow the reference so that its state dicts
load and `add_deformable_conv` can swap these in:
  * ops/dconv-native/src/dconv_native/modules.py (DConv3d, MDConv3d, Spatial*/Temporal*,
    SizeConditioned*/XY*/XYZ*), and
  * network/layers.py:18-313 of the training code (adds the XXZ variants, the
    `size_activation` choices, an optional norm on the predictor input and
    activation checkpointing of the predictor).

The variants differ only in a few class attributes, so one base class implements
them all.  Size-conditioned layers feed the dilation field to the fused
`dyn_dilated_conv3d` kernel by default (`fused_field=True`); with
`fused_field=False` they expand the field with `offsets_from_size_map` exactly as
the reference does (which, like the reference, requires offset_groups == 1).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.modules.utils import _triple
from torch.utils.checkpoint import checkpoint

from .deform_conv import DeformConv3d
from .grid import offsets_from_size_map

_MASK_ACTIVATIONS = {
    "sigmoid": torch.sigmoid,
    "relu": torch.relu,
    "tanh": torch.tanh,
    "linear": lambda t: t,
}


def apply_size_activation(mode, size_map):
    """network/layers.py:171-181."""
    if mode == "elu":
        return F.elu(size_map) + 1
    if mode == "relu":
        return F.relu(size_map + 1)
    if mode == "relu_plus_one":
        return F.relu(size_map + 1e-3) + 1
    if mode == "linear":
        return size_map
    raise ValueError(f"Unexpected size activation mode '{mode}'")


class _DConvBase(nn.Module):
    # variant description (overridden by subclasses)
    modulated = False      # predict a modulation mask (DCNv2)
    field_mode = None      # None: predict 3*G*K offsets; else dilation-field mode "x"/"xy"/"xxz"/"xyz"
    frozen_dims = ()       # offset components (0:z 1:y 2:x) forced to zero (Spatial*/Temporal*)

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 offset_groups=1, bias=True, activation="sigmoid", deform_param_op=nn.Conv3d,
                 size_activation="elu", norm=None, use_checkpoint=False, fused_field=True):
        super().__init__()
        kernel_size = _triple(kernel_size)
        self.num_kernel_points = kernel_size[0] * kernel_size[1] * kernel_size[2]
        self.offset_groups, self.groups = offset_groups, groups
        self.size_activation = size_activation
        self.use_checkpoint = use_checkpoint
        self.fused_field = fused_field
        self.norm = norm
        self.alpha_channels = offset_groups * self.num_kernel_points if self.modulated else 0
        if self.field_mode is None:
            self.offset_channels = 3 * offset_groups * self.num_kernel_points
        else:
            self.offset_channels = {"x": 1, "xy": 2, "xxz": 2, "xyz": 3}[self.field_mode]
        self.deform_params = deform_param_op(in_channels, self._deform_channels(), kernel_size, stride, padding,
                                             dilation, 1, bias)
        self.deform_conv = DeformConv3d(in_channels, out_channels, kernel_size, stride, padding, dilation,
                                        groups, offset_groups, bias)
        self.activation = _MASK_ACTIVATIONS[activation] if isinstance(activation, str) else activation
        # zero-initialised predictor: the layer starts as an ordinary convolution
        nn.init.zeros_(self.deform_params.weight)
        if getattr(self.deform_params, "bias", None) is not None:
            nn.init.zeros_(self.deform_params.bias)

    def _deform_channels(self):
        return self.offset_channels + self.alpha_channels

    def _predict(self, input):
        """-> (offsets or dilation field, activated mask or None)."""
        if self.norm is not None:
            input = self.norm(input)
        raw = self.deform_params(input)
        if self.modulated:
            geo, alpha = torch.split(raw, [self.offset_channels, self.alpha_channels], dim=1)
            alpha = self.activation(alpha)
        else:
            geo, alpha = raw, None
        if self.field_mode is not None:
            geo = apply_size_activation(self.size_activation, geo)
        elif self.frozen_dims:
            geo = geo.clone()
            for d in self.frozen_dims:
                geo[:, d::3] = 0
        return geo, alpha

    def _get_deformation(self, input):
        """Reference-compatible view: always (offsets [B, 3K(*G), ...], mask)."""
        geo, alpha = self._predict(input)
        if self.field_mode is not None:
            geo = offsets_from_size_map(geo, self.field_mode, self.deform_conv.kernel_size,
                                        self.deform_conv.dilation)
        return geo, alpha

    def forward(self, input):
        if self.use_checkpoint and input.requires_grad:
            geo, alpha = checkpoint(self._predict, input, use_reentrant=False)
        else:
            geo, alpha = self._predict(input)
        if self.field_mode is None:
            return self.deform_conv(input, geo, alpha)
        if self.fused_field:
            return self.deform_conv.forward_field(input, geo, alpha, self.field_mode)
        offsets = offsets_from_size_map(geo, self.field_mode, self.deform_conv.kernel_size,
                                        self.deform_conv.dilation)
        return self.deform_conv(input, offsets, alpha)


def _variant(name, **attrs):
    return type(name, (_DConvBase,), dict(attrs, __doc__=f"{name}: {attrs}"))


DConv3d = _variant("DConv3d")
MDConv3d = _variant("MDConv3d", modulated=True)
SpatialDConv3d = _variant("SpatialDConv3d", frozen_dims=(0,))
SpatialMDConv3d = _variant("SpatialMDConv3d", modulated=True, frozen_dims=(0,))
TemporalDConv3d = _variant("TemporalDConv3d", frozen_dims=(1, 2))
TemporalMDConv3d = _variant("TemporalMDConv3d", modulated=True, frozen_dims=(1, 2))
SizeConditionedDConv3d = _variant("SizeConditionedDConv3d", field_mode="x")
XYSizeConditionedDConv3d = _variant("XYSizeConditionedDConv3d", field_mode="xy")
XXZSizeConditionedDConv3d = _variant("XXZSizeConditionedDConv3d", field_mode="xxz")
XYZSizeConditionedDConv3d = _variant("XYZSizeConditionedDConv3d", field_mode="xyz")
SizeConditionedMDConv3d = _variant("SizeConditionedMDConv3d", modulated=True, field_mode="x")
XYSizeConditionedMDConv3d = _variant("XYSizeConditionedMDConv3d", modulated=True, field_mode="xy")
XXZSizeConditionedMDConv3d = _variant("XXZSizeConditionedMDConv3d", modulated=True, field_mode="xxz")
XYZSizeConditionedMDConv3d = _variant("XYZSizeConditionedMDConv3d", modulated=True, field_mode="xyz")

__all__ = [n for n, v in list(globals().items()) if isinstance(v, type) and issubclass(v, _DConvBase)]
