"""Stand-in for the reference's compiled `fast_depthwise_conv3d._ops`
(ops/fast-depthwise-conv3d/csrc/python_bindings.cpp:4-6):
`depthwise_separable_conv3d(input, weight, bias, stride, padding, dilation)` with the
autograd of DepthwiseConv3dFunction (csrc/grouped_conv3d.h:29-106)."""
import ctypes

import torch
from torch.autograd.function import once_differentiable
from torch.nn.modules.utils import _triple

from .. import _lib


class _DepthwiseConv3dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias, stride, padding, dilation):
        if not input.is_cuda or not weight.is_cuda:
            raise RuntimeError("depthwise_separable_conv3d expects CUDA tensors")
        if input.device != weight.device or (bias is not None and bias.device != input.device):
            raise RuntimeError("expects input and weight tensors to be on the same device.")
        unbatched = input.dim() == 4
        x = input.unsqueeze(0) if unbatched else input
        if x.dim() != 5:
            raise RuntimeError(f"Input dimension should be 4D or 5D, got {input.dim()}D")
        if weight.dim() != 5:
            raise RuntimeError(f"Weight dimension should be 5D, got {weight.dim()}D")
        if weight.size(1) != 1:
            raise RuntimeError(f"Depthwise weight should have in_channels=1, got {weight.size(1)}")
        if weight.size(0) % x.size(1) != 0:
            raise RuntimeError("Depthwise out channels should be a multiple of in channels, got "
                               f"{weight.size(0)} and {x.size(1)}")
        if bias is not None and (bias.dim() != 1 or bias.size(0) != weight.size(0)):
            raise RuntimeError(f"Bias length should be equal to out_channels, got {tuple(bias.shape)} and {weight.size(0)}")
        if weight.dtype != x.dtype or (bias is not None and bias.dtype != x.dtype):
            raise RuntimeError("input, weight and bias must have the same dtype")
        x, w = x.contiguous(), weight.contiguous()
        b = None if bias is None else bias.contiguous()
        desc = _lib.make_desc(x, w, stride, padding, dilation, x.shape[1], 1)
        out_dims = _lib.output_dims(desc, "depthwise_separable_conv3d")
        L = _lib.lib()
        with torch.cuda.device(x.device):
            y = torch.empty((x.shape[0], w.shape[0]) + out_dims, dtype=x.dtype, device=x.device)
            _lib.check(L.d2c_depthwise_conv3d_fwd(ctypes.byref(desc), _lib.ptr(x), _lib.ptr(w), _lib.ptr(b),
                                                  _lib.ptr(y), _lib.stream_of(x)), "depthwise_separable_conv3d forward")
        ctx.save_for_backward(x, w, b)
        ctx.desc, ctx.unbatched = desc, unbatched
        return y.squeeze(0) if unbatched else y

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        x, w, b = ctx.saved_tensors
        desc = ctx.desc
        gy = (grad_out.unsqueeze(0) if ctx.unbatched else grad_out).contiguous()
        need_x, need_w, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1], b is not None and ctx.needs_input_grad[2]
        L = _lib.lib()
        with torch.cuda.device(x.device):
            gx = torch.empty_like(x) if need_x else None
            gw = torch.empty_like(w) if need_w else None
            gb = torch.empty_like(b) if need_b else None
            ws, ws_bytes = _lib.workspace(_lib.OP_DW_BWD, desc, x.device) if need_w else (None, 0)
            _lib.check(L.d2c_depthwise_conv3d_bwd(
                ctypes.byref(desc), _lib.ptr(gy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(gx), _lib.ptr(gw), _lib.ptr(gb),
                _lib.ptr(ws), ws_bytes, _lib.stream_of(x)), "depthwise_separable_conv3d backward")
        if gx is not None and ctx.unbatched:
            gx = gx.squeeze(0)
        return gx, gw, gb, None, None, None


def depthwise_separable_conv3d(input, weight, bias, stride, padding, dilation):
    return _DepthwiseConv3dFunction.apply(input, weight, bias, tuple(_triple(stride)), tuple(_triple(padding)),
                                          tuple(_triple(dilation)))
