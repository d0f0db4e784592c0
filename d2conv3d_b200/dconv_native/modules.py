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

from . import _ops
from .deform_conv import DeformConv3d
from .grid import offsets_from_size_map

_MASK_ACTIVATIONS = {
    "sigmoid": torch.sigmoid,
    "relu": torch.relu,
    "tanh": torch.tanh,
    "linear": lambda t: t,
    "none": lambda t: t,
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


# Positional arguments after `activation`: the package's modules.py continues with (deform_param_op), the
# training code's network/layers.py with (init, norm_type, norm_groups, size_activation, deform_param_op).
_LAYERS_PY_ORDER = ("init", "norm_type", "norm_groups", "size_activation", "deform_param_op")


class _DConvBase(nn.Module):
    """Constructor: the ten leading arguments of both reference classes, then either reference's remaining ones
    (positionally: a string in 11th place means network/layers.py's order, anything else the package's
    `deform_param_op`), all of them also accepted as keywords:

      init             "zero" (default) | "random" (modulated layers only: network/layers.py:122-132)
      norm_type        "none" | "GroupNorm" | "BatchNorm": a norm on the predictor's input (layers.py:37-44)
      norm_groups      groups of that GroupNorm
      size_activation  "elu" | "relu" | "relu_plus_one" | "linear" (layers.py:171-181)
      deform_param_op  class of the predictor, or a ready nn.Module instance (then used as is, not initialised)

    and four that only this package has: `norm` (a ready norm module instead of norm_type), `use_checkpoint`
    (recompute the predictor in the backward, what layers.py:99 always does), `fused_field` (hand the dilation field
    to the kernels instead of expanding it to 3*K offset channels) and `fused_head` (default True: the predictor's
    raw output goes to the op as it is -- split, mask activation and size activation happen inside the kernels,
    forward and backward; taken when the activation is one of the named ones, the tensors are CUDA fp32 / fp64 and
    neither `use_checkpoint` nor frozen offset components are in play, otherwise the unfused path runs)."""

    # variant description (overridden by subclasses)
    modulated = False      # predict a modulation mask (DCNv2)
    field_mode = None      # None: predict 3*G*K offsets; else dilation-field mode "x"/"xy"/"xxz"/"xyz"
    frozen_dims = ()       # offset components (0:z 1:y 2:x) forced to zero (Spatial*/Temporal*)

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 offset_groups=1, bias=True, activation="sigmoid", *extra, **kw):
        super().__init__()
        if extra:
            names = _LAYERS_PY_ORDER if isinstance(extra[0], str) else ("deform_param_op",)
            if len(extra) > len(names):
                raise TypeError(f"too many positional arguments ({10 + len(extra)})")
            for n, v in zip(names, extra):
                if n in kw:
                    raise TypeError(f"got multiple values for argument '{n}'")
                kw[n] = v
        init = kw.pop("init", "zero")
        norm_type = kw.pop("norm_type", "none")
        norm_groups = kw.pop("norm_groups", 1)
        size_activation = kw.pop("size_activation", "elu")
        deform_param_op = kw.pop("deform_param_op", nn.Conv3d)
        norm = kw.pop("norm", None)
        use_checkpoint = kw.pop("use_checkpoint", False)
        fused_field = kw.pop("fused_field", True)
        fused_head = kw.pop("fused_head", True)
        if kw:
            raise TypeError(f"unexpected keyword argument(s): {sorted(kw)}")

        kernel_size = _triple(kernel_size)
        self.num_kernel_points = kernel_size[0] * kernel_size[1] * kernel_size[2]
        self.offset_groups, self.groups = offset_groups, groups
        self.size_activation = size_activation
        self.use_checkpoint = use_checkpoint
        self.fused_field = fused_field
        self.fused_head = fused_head
        self._mask_act_name = activation if isinstance(activation, str) else None
        if norm_type not in ("BatchNorm", "GroupNorm", "none"):
            raise ValueError(f"Unexpected norm_type: '{norm_type}'")
        if norm is None and norm_type == "GroupNorm":
            norm = nn.GroupNorm(norm_groups, in_channels)
        elif norm is None and norm_type == "BatchNorm":
            norm = nn.BatchNorm3d(in_channels)
        self.norm = norm
        self.alpha_channels = offset_groups * self.num_kernel_points if self.modulated else 0
        if self.field_mode is None:
            self.offset_channels = 3 * offset_groups * self.num_kernel_points
        else:
            self.offset_channels = {"x": 1, "xy": 2, "xxz": 2, "xyz": 3}[self.field_mode]
        if isinstance(deform_param_op, nn.Module):
            self.deform_params = deform_param_op
        else:
            self.deform_params = deform_param_op(in_channels, self._deform_channels(), kernel_size, stride, padding,
                                                 dilation, 1, bias)
        self.deform_conv = DeformConv3d(in_channels, out_channels, kernel_size, stride, padding, dilation,
                                        groups, offset_groups, bias)
        self.activation = _MASK_ACTIVATIONS[activation] if isinstance(activation, str) else activation
        if not isinstance(deform_param_op, nn.Module):
            self._init_deform_params(activation, init)

    def _init_deform_params(self, activation, init):
        """network/layers.py:78-86 (offset-only layers) and :122-132 (modulated layers)."""
        w = self.deform_params.weight
        if init == "zero":
            # the layer starts as an ordinary convolution (times the activation of 0 when modulated)
            nn.init.zeros_(w)
        elif init == "random" and self.modulated:
            # the reference re-draws the modulation rows only; the geometry rows keep the predictor's own init
            with torch.no_grad():
                if activation in ("sigmoid", "tanh"):
                    nn.init.xavier_normal_(w[self.offset_channels:])
                else:
                    nn.init.kaiming_normal_(w[self.offset_channels:])
        else:
            raise ValueError(f"init scheme {init} not supported")
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

    def _can_fuse_head(self, input):
        return (self.fused_head and input.is_cuda and input.dtype in (torch.float32, torch.float64)
                and not self.frozen_dims and not (self.use_checkpoint and input.requires_grad)
                and (not self.modulated or self._mask_act_name is not None)
                and (self.field_mode is None or self.fused_field)
                and self.deform_conv.weight.dtype == input.dtype)

    def forward(self, input):
        if self._can_fuse_head(input):
            raw = self.deform_params(input if self.norm is None else self.norm(input))
            dc = self.deform_conv
            # a half-precision predictor output (autocast) is up-cast, as the reference's front-end does
            return _ops.deform_conv3d_head(input, raw.to(input.dtype), dc.weight, dc.bias, self.field_mode,
                                           self.modulated, self._mask_act_name or "linear", self.size_activation,
                                           dc.stride, dc.padding, dc.dilation, dc.groups, dc.offset_groups)
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
