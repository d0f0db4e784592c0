"""Random-init, configuration-free version of the D2Conv3D segmentation decoder, so that the decoder-inference
configuration of the benchmark (four ir-CSN pyramid levels -> mask logits) runs end to end on this package's
operators plus stock PyTorch convolutions / norms / interpolation.

Structure follows the reference:
  * global-convolution bridge on the coarsest level: two separable 7-tap branches, (1,7,1)->(1,1,7) and
    (1,1,7)->(1,7,1), summed (network/modules/bridging.py:12-29);
  * a two-conv residual on top of it and three refine blocks, coarse to fine
    (network/segmentation/encoder_decoder.py:106-150);
  * a refine block = conv -> activation -> norm three times on the skip feature (the last two as a residual),
    add the trilinearly up-sampled coarser map, two more conv units as a residual
    (network/modules/refinement.py:26-64);
  * prediction conv on relu(m1), up-sampled x4 in height and width (encoder_decoder.py:153-164).
The 3x3x3 convolutions of the refine blocks are the deformable layer type given by `conv` (default: the
dilation-field + modulation-mask layer, "XYZSizeConditionedDCNv2" in the reference's naming), swapped in with the
package's `add_deformable_conv`, exactly how the reference converts its decoder (encoder_decoder.py:132-141).

Clips are independent: sharding a batch of clips over GPUs needs no communication (`shard_clips`).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .dconv_native.util import add_deformable_conv


class GlobalConv3d(nn.Module):
    """Separable large-kernel bridge: (1,k,1) then (1,1,k), plus (1,1,k) then (1,k,1)."""

    def __init__(self, in_channels, out_channels, k=7, mid_channels=256):
        super().__init__()
        p = k // 2
        self.conv_l1 = nn.Conv3d(in_channels, mid_channels, (1, k, 1), padding=(0, p, 0))
        self.conv_l2 = nn.Conv3d(mid_channels, out_channels, (1, 1, k), padding=(0, 0, p))
        self.conv_r1 = nn.Conv3d(in_channels, mid_channels, (1, 1, k), padding=(0, 0, p))
        self.conv_r2 = nn.Conv3d(mid_channels, out_channels, (1, k, 1), padding=(0, p, 0))

    def forward(self, x):
        return self.conv_l2(self.conv_l1(x)) + self.conv_r2(self.conv_r1(x))


class ConvActNorm(nn.Sequential):
    """conv -> activation -> norm, in this order (refinement.py:38-43); GroupNorm with one group.  Same three
    sub-modules (and state-dict keys) as the reference's nn.Sequential.  The ReLU + GroupNorm tail (forward and
    backward) runs as the library's fused streaming kernels (fp32 CUDA tensors only): PyTorch's GroupNorm reduces
    each (clip, group) row in ONE thread block, which for one group of 50 M elements takes 19 ms per layer and
    was 85 % of the decoder's inference time."""

    def __init__(self, cin, cout):
        super().__init__(nn.Conv3d(cin, cout, 3, padding=1), nn.ReLU(), nn.GroupNorm(1, cout))

    def forward(self, x):
        from . import _lib
        y = self[0](x)
        norm = self[2]
        # no eager stand-in: act_group_norm raises for anything but an fp32 CUDA tensor
        return _lib.act_group_norm(y, norm.weight, norm.bias, norm.num_groups, norm.eps, relu=True)


def _unit(cin, cout):
    return ConvActNorm(cin, cout)


class Refine3d(nn.Module):
    def __init__(self, in_channels, channels):
        super().__init__()
        self.convFS1 = _unit(in_channels, channels)
        self.convFS2 = _unit(channels, channels)
        self.convFS3 = _unit(channels, channels)
        self.convMM1 = _unit(channels, channels)
        self.convMM2 = _unit(channels, channels)

    def forward(self, feature, coarser):
        s = self.convFS1(feature)
        s = s + self.convFS3(self.convFS2(s))
        m = s + F.interpolate(coarser, size=s.shape[-3:], mode="trilinear", align_corners=False)
        return m + self.convMM2(self.convMM1(m))


class Decoder(nn.Module):
    """widths: channels of the four pyramid levels, fine to coarse.  conv: None for plain convolutions, or a
    version name understood by add_deformable_conv for the refine blocks' 3x3x3 convolutions."""

    def __init__(self, widths=(256, 512, 1024, 2048), channels=256, num_classes=2,
                 conv="XYZSizeConditionedDCNv2", offset_groups=8):
        super().__init__()
        self.gc = GlobalConv3d(widths[3], channels, mid_channels=channels)
        self.convG1 = nn.Conv3d(channels, channels, 3, padding=1)
        self.convG2 = nn.Conv3d(channels, channels, 3, padding=1)
        self.rf3 = Refine3d(widths[2], channels)
        self.rf2 = Refine3d(widths[1], channels)
        self.rf1 = Refine3d(widths[0], channels)
        self.pred = nn.Conv3d(channels, num_classes, 3, padding=1)
        self.converted = 0
        if conv is not None:
            for name in ("rf3", "rf2", "rf1"):
                block, n = add_deformable_conv(getattr(self, name), version=conv, offset_groups=offset_groups)
                setattr(self, name, block)
                self.converted += n

    def forward(self, e1, e2, e3, e4):
        x = self.gc(e4)
        m4 = x + self.convG2(F.relu(self.convG1(F.relu(x))))
        m3 = self.rf3(e3, m4)
        m2 = self.rf2(e2, m3)
        m1 = self.rf1(e1, m2)
        p1 = self.pred(F.relu(m1))
        return F.interpolate(p1, scale_factor=(1, 4, 4), mode="trilinear")


def pyramid_shapes(clips, frames=8, height=480, width=854, widths=(256, 512, 1024, 2048)):
    """Feature shapes of an ir-CSN backbone for `clips` clips of `frames` frames: strides 4, 8, 16, 32 in
    height / width (rounded up), the frame count kept (the benchmark's convention)."""
    out = []
    for c, s in zip(widths, (4, 8, 16, 32)):
        out.append((clips, c, frames, -(-height // s), -(-width // s)))
    return out
