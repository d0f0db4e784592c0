"""`DepthwiseConv3d`, as ops/fast-depthwise-conv3d/src/fast_depthwise_conv3d/conv.py:7-22:
an nn.Conv3d whose groups equal its input channels, evaluated by the depthwise kernels
of libd2conv3d.so.  Parameters are cast to the input's dtype (so fp16 inputs under
autocast give fp16 outputs); non-zero padding modes pad explicitly first."""
import torch.nn as nn
import torch.nn.functional as F

from . import _ops


class DepthwiseConv3d(nn.Conv3d):
    def __init__(self, in_channels, out_channels, kernel_size=1, stride=1, padding=0, dilation=1, groups=None,
                 bias=True, padding_mode="zeros"):
        # `groups` is accepted for signature compatibility and ignored: always depthwise
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, in_channels, bias,
                         padding_mode)

    def forward(self, input):
        weight = self.weight.to(dtype=input.dtype)
        bias = None if self.bias is None else self.bias.to(dtype=input.dtype)
        padding = self.padding
        if self.padding_mode != "zeros":
            input = F.pad(input, self._reversed_padding_repeated_twice, mode=self.padding_mode)
            padding = (0, 0, 0)
        return _ops.depthwise_separable_conv3d(input, weight, bias, self.stride, padding, self.dilation)
