"""Conv3d -> deformable layer replacement, as ops/dconv-native/src/dconv_native/util.py
(`add_deformable_conv(module, version=..., offset_groups=..., activation=...,
replace_1x1_kernels=...)`, returning (module, number_of_replacements))."""
import torch.nn as nn

from . import modules as _m
from .modules import *  # noqa: F401,F403  (the reference re-exports the layer classes here)

_VERSIONS = {
    "DCNv1": _m.DConv3d, "DCNv2": _m.MDConv3d,
    "SpatialDCNv1": _m.SpatialDConv3d, "SpatialDCNv2": _m.SpatialMDConv3d,
    "TemporalDCNv1": _m.TemporalDConv3d, "TemporalDCNv2": _m.TemporalMDConv3d,
    "SizeConditionedDCNv1": _m.SizeConditionedDConv3d, "SizeConditionedDCNv2": _m.SizeConditionedMDConv3d,
    "XYSizeConditionedDCNv1": _m.XYSizeConditionedDConv3d, "XYSizeConditionedDCNv2": _m.XYSizeConditionedMDConv3d,
    "XXZSizeConditionedDCNv1": _m.XXZSizeConditionedDConv3d, "XXZSizeConditionedDCNv2": _m.XXZSizeConditionedMDConv3d,
    "XYZSizeConditionedDCNv1": _m.XYZSizeConditionedDConv3d, "XYZSizeConditionedDCNv2": _m.XYZSizeConditionedMDConv3d,
}


def replace_module(replacement_func, replaced_cls, module, **kwargs):
    """Depth-first replacement of every `replaced_cls` instance; returns (module, count)."""
    count = 0
    result = module
    if isinstance(module, replaced_cls):
        result = replacement_func(module, **kwargs)
        count += int(result is not module)
    for name, child in list(module.named_children()):
        new_child, n = replace_module(replacement_func, replaced_cls, child, **kwargs)
        result.add_module(name, new_child)
        count += n
    return result, count


def dconv_replace_layer(conv, **kwargs):
    if conv.kernel_size == (1, 1, 1) and not kwargs.get("replace_1x1_kernels"):
        return conv
    cls = _VERSIONS[kwargs["version"]]
    layer = cls(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding, conv.dilation,
                conv.groups, kwargs.get("offset_groups", 1), conv.bias is not None,
                kwargs.get("activation", "sigmoid"))
    layer = layer.to(device=conv.weight.device, dtype=conv.weight.dtype)
    layer.deform_conv.weight.data = conv.weight.data.detach()
    if conv.bias is not None:
        layer.deform_conv.bias.data = conv.bias.data.detach()
    return layer


def add_deformable_conv(module, **kwargs):
    return replace_module(dconv_replace_layer, nn.Conv3d, module, **kwargs)
