"""CPU-only checks of the Python mirror of the reference's packages: names, signatures,
parameter shapes / initialisation, module replacement, and error behaviour without a GPU."""
import inspect

import numpy as np
import pytest
import torch
import torch.nn as nn

import d2conv3d_b200
from d2conv3d_b200 import dconv_native, fast_depthwise_conv3d
from d2conv3d_b200.dconv_native import modules, util
from d2conv3d_b200.dconv_native.grid import offsets_from_size_map
from tests._util import size_map_cases


def test_public_names_of_reference_packages():
    for n in ["deform_conv1d", "deform_conv3d", "DeformConv1d", "DeformConv3d", "DConv3d", "MDConv3d",
              "SizeConditionedDConv3d", "SizeConditionedMDConv3d"]:
        assert n in dconv_native.__all__ and hasattr(dconv_native, n)
    assert hasattr(dconv_native.deform_conv, "DeformConvNd")
    assert callable(dconv_native._ops.deform_conv3d)
    assert callable(dconv_native._ops.config.get_max_intermediate_elements)
    assert callable(fast_depthwise_conv3d._ops.depthwise_separable_conv3d)
    assert issubclass(fast_depthwise_conv3d.DepthwiseConv3d, nn.Conv3d)


def test_signatures_match_reference():
    sig = inspect.signature(dconv_native.deform_conv3d)
    assert list(sig.parameters) == ["input", "offset", "alpha", "weight", "bias", "stride", "padding", "dilation",
                                    "n_weight_groups", "n_offset_groups"]
    sig = inspect.signature(dconv_native._ops.deform_conv3d)
    assert len(sig.parameters) == 16
    sig = inspect.signature(dconv_native.DeformConv3d.__init__)
    assert list(sig.parameters)[1:] == ["in_channels", "out_channels", "kernel_size", "stride", "padding",
                                        "dilation", "groups", "offset_groups", "bias"]
    sig = inspect.signature(fast_depthwise_conv3d.DepthwiseConv3d.__init__)
    assert list(sig.parameters)[1:] == ["in_channels", "out_channels", "kernel_size", "stride", "padding",
                                        "dilation", "groups", "bias", "padding_mode"]


def test_deform_conv3d_module_parameters():
    m = dconv_native.DeformConv3d(12, 6, (3, 5, 3), groups=3, offset_groups=2)
    assert tuple(m.weight.shape) == (6, 4, 3, 5, 3) and tuple(m.bias.shape) == (6,)
    assert m.stride == (1, 1, 1) and m.padding == (0, 0, 0) and m.dilation == (1, 1, 1)
    fan_in = 4 * 45
    assert m.bias.abs().max() <= 1 / np.sqrt(fan_in)
    assert dconv_native.DeformConv3d(4, 4, 3, bias=False).bias is None
    with pytest.raises(ValueError):
        dconv_native.DeformConv3d(5, 4, 3, groups=2)
    with pytest.raises(ValueError):
        dconv_native.DeformConv3d(6, 4, 3, offset_groups=4)


@pytest.mark.parametrize("cls,channels", [
    ("DConv3d", 3 * 2 * 27), ("MDConv3d", 4 * 2 * 27), ("SpatialMDConv3d", 4 * 2 * 27),
    ("SizeConditionedDConv3d", 1), ("XYSizeConditionedDConv3d", 2), ("XXZSizeConditionedDConv3d", 2),
    ("XYZSizeConditionedDConv3d", 3), ("SizeConditionedMDConv3d", 1 + 2 * 27),
    ("XYZSizeConditionedMDConv3d", 3 + 2 * 27)])
def test_layer_variants_predictor_channels_and_zero_init(cls, channels):
    layer = getattr(modules, cls)(4, 8, 3, padding=1, offset_groups=2)
    assert layer.deform_params.out_channels == channels
    assert layer.deform_params.weight.abs().sum() == 0 and layer.deform_params.bias.abs().sum() == 0
    assert isinstance(layer.deform_conv, dconv_native.DeformConv3d)
    assert layer.deform_conv.offset_groups == 2


def test_get_deformation_on_cpu_matches_reference_semantics():
    layer = modules.SizeConditionedMDConv3d(3, 4, 3, padding=1)
    x = torch.randn(1, 3, 4, 5, 5)
    offsets, alpha = layer._get_deformation(x)
    assert tuple(offsets.shape) == (1, 81, 4, 5, 5) and tuple(alpha.shape) == (1, 27, 4, 5, 5)
    assert offsets.abs().max() == 0          # elu(0)+1 = 1 -> zero offsets
    assert torch.all(alpha == 0.5)           # sigmoid(0)
    layer = modules.TemporalDConv3d(3, 4, 3, padding=1)
    nn.init.normal_(layer.deform_params.weight)
    offsets, alpha = layer._get_deformation(x)
    assert alpha is None
    assert offsets[:, 1::3].abs().max() == 0 and offsets[:, 2::3].abs().max() == 0 and offsets[:, 0::3].abs().max() > 0


def test_layer_constructor_accepts_both_reference_signatures():
    """The package's modules.py (ops/dconv-native/src/dconv_native/modules.py:17-19) continues after `activation`
    with deform_param_op; the training code's network/layers.py:27-30 with init, norm_type, norm_groups,
    size_activation, deform_param_op.  Both call styles, positional and keyword, must work."""
    # network/layers.py keywords
    layer = modules.MDConv3d(8, 8, 3, padding=1, init="zero", norm_type="GroupNorm", norm_groups=2,
                             size_activation="relu", deform_param_op=nn.Conv3d, activation="none")
    assert isinstance(layer.norm, nn.GroupNorm) and layer.norm.num_groups == 2 and layer.size_activation == "relu"
    assert layer.activation(torch.tensor(-3.0)) == -3.0                     # "none" = identity
    assert isinstance(modules.DConv3d(8, 8, 3, norm_type="BatchNorm").norm, nn.BatchNorm3d)
    with pytest.raises(ValueError):
        modules.DConv3d(8, 8, 3, norm_type="LayerNorm")
    # layers.py positional order: (..., activation, init, norm_type, norm_groups, size_activation, deform_param_op)
    layer = modules.XYZSizeConditionedMDConv3d(8, 8, 3, 1, 1, 1, 1, 2, True, "sigmoid", "zero", "GroupNorm", 4,
                                                "relu_plus_one", nn.Conv3d)
    assert layer.norm.num_groups == 4 and layer.size_activation == "relu_plus_one"
    # package order: (..., activation, deform_param_op)
    made = []

    def factory(*a):
        made.append(a)
        return nn.Conv3d(*a)
    layer = modules.DConv3d(8, 8, 3, 1, 1, 1, 1, 1, True, "sigmoid", factory)
    assert made and made[0][1] == 81
    # a ready module instance is used as is and not re-initialised
    pred = nn.Conv3d(8, 4 * 27, 3, padding=1)
    nn.init.constant_(pred.weight, 0.25)
    layer = modules.MDConv3d(8, 8, 3, padding=1, deform_param_op=pred)
    assert layer.deform_params is pred and torch.all(pred.weight == 0.25)
    with pytest.raises(TypeError):
        modules.DConv3d(8, 8, 3, bogus=1)


def test_layer_init_schemes_follow_the_training_code():
    """network/layers.py:78-86,122-132: 'zero' for every layer; 'random' only for modulated layers, where it re-draws
    the modulation rows of the predictor and zeroes its bias."""
    torch.manual_seed(0)
    layer = modules.MDConv3d(8, 8, 3, padding=1, init="random")
    w = layer.deform_params.weight
    assert w[layer.offset_channels:].abs().sum() > 0 and layer.deform_params.bias.abs().sum() == 0
    layer = modules.XYZSizeConditionedMDConv3d(8, 8, 3, padding=1, init="random", activation="relu")
    assert layer.deform_params.weight[3:].abs().sum() > 0
    with pytest.raises(ValueError):
        modules.DConv3d(8, 8, 3, init="random")
    with pytest.raises(ValueError):
        modules.MDConv3d(8, 8, 3, init="orthogonal")


def test_add_deformable_conv_replaces_conv3d():
    net = nn.Sequential(nn.Conv3d(4, 8, 3, padding=1), nn.ReLU(), nn.Sequential(nn.Conv3d(8, 8, 1), nn.Conv3d(8, 4, 3, bias=False)))
    w0 = net[0].weight.data.clone()
    new, n = util.add_deformable_conv(net, version="XYZSizeConditionedDCNv2", offset_groups=2)
    assert n == 2
    assert isinstance(new[0], modules.XYZSizeConditionedMDConv3d) and isinstance(new[2][0], nn.Conv3d)
    assert torch.equal(new[0].deform_conv.weight.data, w0)
    assert new[2][1].deform_conv.bias is None
    new, n = util.add_deformable_conv(nn.Sequential(nn.Conv3d(8, 8, 1)), version="DCNv1", replace_1x1_kernels=True)
    assert n == 1


def test_grid_matches_reference_outputs_bit_exact():
    s = size_map_cases()
    for n in s["names"]:
        kd = [int(v) for v in s[f"{n}/kd"]]
        mode = str(n).split("_")[0]
        o = offsets_from_size_map(torch.from_numpy(s[f"{n}/size_map"]), mode, tuple(kd[:3]), tuple(kd[3:]))
        assert np.array_equal(o.numpy(), s[f"{n}/offsets"]), n
    # the older signature infers the mode from the channel count
    sm = torch.rand(1, 2, 2, 3, 3) + 1
    assert torch.equal(offsets_from_size_map(sm, (3, 3, 3), (1, 1, 1)), offsets_from_size_map(sm, "xy"))
    with pytest.raises(ValueError):
        offsets_from_size_map(torch.rand(1, 4, 2, 2, 2))


def test_cpu_tensors_are_rejected_like_the_reference():
    x = torch.randn(1, 2, 3, 3, 3)
    off = torch.zeros(1, 81, 1, 1, 1)
    w = torch.randn(2, 2, 3, 3, 3)
    with pytest.raises(RuntimeError, match=r"is_cuda"):
        dconv_native.deform_conv3d(x, off, None, w)
    with pytest.raises(RuntimeError):
        fast_depthwise_conv3d.DepthwiseConv3d(2, 2, 3)(x)
    with pytest.raises(RuntimeError, match=r"is_cuda"):      # the 1-D op runs on the 3-D kernels: same check
        dconv_native.deform_conv1d(torch.randn(1, 2, 5), torch.zeros(1, 3, 3), None, torch.randn(2, 2, 3))


def test_install_as_dropin():
    d2conv3d_b200.install_as_dropin()
    import dconv_native as top
    import dconv_native._ops as ops
    from fast_depthwise_conv3d import DepthwiseConv3d
    assert top is dconv_native and ops is dconv_native._ops
    assert DepthwiseConv3d is fast_depthwise_conv3d.DepthwiseConv3d
