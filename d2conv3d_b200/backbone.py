"""ir-CSN bottleneck block (channel-separated ResNet, "interaction-reduced" variant) around this package's
depthwise conv3d: 1x1x1 conv -> BN -> ReLU -> depthwise 3x3x3 (no bias) -> BN -> ReLU -> 1x1x1 conv (x4
channels) -> BN, residual add, ReLU -- the block of the reference's backbone (network/backbone/resnet.py:59-118),
written free of its global configuration so the depthwise kernels can be measured where they are used.
Optional activation checkpointing as in the reference (:113-117)."""
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .fast_depthwise_conv3d import DepthwiseConv3d


class IrBottleneck3d(nn.Module):
    expansion = 4

    def __init__(self, in_channels, channels, stride=1, dilation=1, downsample=None, use_checkpoint=False,
                 depthwise=DepthwiseConv3d):
        super().__init__()
        self.conv1 = nn.Conv3d(in_channels, channels, 1, bias=False)
        self.bn1 = nn.BatchNorm3d(channels)
        self.conv2 = depthwise(channels, channels, kernel_size=3, stride=stride, padding=dilation, dilation=dilation,
                               groups=channels, bias=False)
        self.bn2 = nn.BatchNorm3d(channels)
        self.conv3 = nn.Conv3d(channels, channels * self.expansion, 1, bias=False)
        self.bn3 = nn.BatchNorm3d(channels * self.expansion)
        self.downsample = downsample
        self.use_checkpoint = use_checkpoint

    def _body(self, x):
        out = self.bn1(self.conv1(x)).relu()
        out = self.bn2(self.conv2(out)).relu()
        out = self.bn3(self.conv3(out))
        if self.downsample is not None:
            x = self.downsample(x)
        return (out + x).relu()

    def forward(self, x):
        if self.use_checkpoint and x.requires_grad:
            return checkpoint(self._body, x, use_reentrant=False)
        return self._body(x)
