"""Stand-in for the reference's compiled module `dconv_native._ops`
(ops/dconv-native/csrc/ops/dconv.cpp:6-12): `deform_conv3d`, `deform_conv1d`
and the `config` sub-namespace, with the same positional signatures.  The work is
done by libd2conv3d.so through the C ABI; autograd is a Python Function that
mirrors DeformConv3dFunction (csrc/ops/dconv3d.h:70-186).
"""
import ctypes
import types

import torch
from torch.autograd.function import once_differentiable

from .. import _lib


class _BackwardState:
    """Event recorded by the most recent deformable backward once grad_weight and grad_bias were final."""
    params_ready = None


def params_ready_event():
    """The torch.cuda.Event that the most recent `deform_conv3d` / `dyn_dilated_conv3d` backward of this process
    recorded as soon as its parameter gradients (grad_weight, grad_bias) were final -- on the tensor-core tier
    before the data-side gradients are computed.  A data-parallel trainer makes a side stream wait for it and
    all-reduces the parameter gradients there (d2conv3d_b200.sharding.all_reduce_param_grads_overlapped), which
    hides the collective under the rest of the backward.  None before the first backward."""
    return _BackwardState.params_ready


def _new_event(stream):
    ev = torch.cuda.Event()
    ev.record(stream)                  # creates the underlying CUDA event; the library records it again later
    return ev


def _will_differentiate(*tensors):
    """Whether autograd is recording this call -- evaluated where the op is CALLED: inside Function.forward grad mode
    is always off and ctx.needs_input_grad reports requires_grad even under torch.no_grad(), so an inference pass over
    a model with trainable weights would otherwise look like a training pass (and keep samples it never uses)."""
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def _require(cond, expr):
    # TORCH_CHECK(expr) of the reference raises RuntimeError("Expected <expr> to be true ...")
    if not cond:
        raise RuntimeError(f"Expected {expr} to be true, but got false.")


def _sanity_check(input, offset, alpha, weight, bias):
    """SANITY_CHECK_DCONV_INPUTS, csrc/ops/dconv_gpu_common.h:26-44 (after .contiguous())."""
    _require(input.dim() == 5, "input.ndimension() == ((3) + 2)")
    _require(offset.dim() == 5, "offset.ndimension() == ((3) + 2)")
    if alpha is not None:
        _require(alpha.dim() == 5, "alpha.ndimension() == ((3) + 2)")
    _require(weight.dim() == 5, "weight.ndimension() == ((3) + 2)")
    if bias is not None:
        _require(bias.dim() == 1, "bias.ndimension() == 1")
    _require(input.is_cuda, "input.device().is_cuda()")
    _require(offset.is_cuda, "offset.device().is_cuda()")
    if alpha is not None:
        _require(alpha.is_cuda, "alpha.device().is_cuda()")
    _require(weight.is_cuda, "weight.device().is_cuda()")
    if bias is not None:
        _require(bias.is_cuda, "bias.device().is_cuda()")
    _require(offset.size(0) == input.size(0), "offset.size(0) == input.size(0)")
    if alpha is not None:
        _require(alpha.size(0) == input.size(0), "alpha.size(0) == input.size(0)")
    for t in (offset, alpha, weight, bias):
        if t is not None and t.dtype != input.dtype:
            raise RuntimeError(f"expected scalar type {input.dtype} but found {t.dtype}")
    if input.dtype not in (torch.float32, torch.float64):
        raise RuntimeError(f'"deform_conv3d" not implemented for \'{input.dtype}\'')


def _check_groups(input, weight, bias, groups):
    _require(weight.size(1) * groups == input.size(1), "weight.size(1) * (n_weight_groups) == input.size(1)")
    if bias is not None:
        _require(bias.size(0) == weight.size(0), "bias.size(0) == weight.size(0)")


class _DeformConv3dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, offset, alpha, weight, bias, sd, sh, sw, pd, ph, pw, dd, dh, dw,
                groups, offset_groups, differentiated):
        input, offset, weight = input.contiguous(), offset.contiguous(), weight.contiguous()
        alpha = None if alpha is None else alpha.contiguous()
        bias = None if bias is None else bias.contiguous()
        _sanity_check(input, offset, alpha, weight, bias)
        _check_groups(input, weight, bias, groups)
        desc = _lib.make_desc(input, weight, (sd, sh, sw), (pd, ph, pw), (dd, dh, dw), groups, offset_groups)
        L = _lib.lib()
        od = (ctypes.c_int64 * 4)(*offset.shape[1:])
        md = None if alpha is None else (ctypes.c_int64 * 4)(*alpha.shape[1:])
        _lib.check(L.d2c_deform_conv3d_check(ctypes.byref(desc), od, md), "deform_conv3d")
        out_dims = _lib.output_dims(desc, "deform_conv3d")
        with torch.cuda.device(input.device):
            y = torch.empty((input.shape[0], weight.shape[0]) + out_dims, dtype=input.dtype, device=input.device)
            ws, ws_bytes = _lib.workspace(_lib.OP_DEFORM_FWD, desc, input.device)
            cache = _lib.SampleCache.for_forward(desc, input.device, differentiated)
            _lib.check(L.d2c_deform_conv3d_fwd(
                ctypes.byref(desc), _lib.ptr(input), _lib.ptr(offset), _lib.ptr(alpha), _lib.ptr(weight),
                _lib.ptr(bias), _lib.ptr(y), _lib.ptr(ws), ws_bytes, _lib.stream_of(input)), "deform_conv3d forward")
        ctx.save_for_backward(input, offset, alpha, weight, bias)
        ctx.desc = desc
        ctx.sample_cache = _lib.finish_forward_cache(cache)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        input, offset, alpha, weight, bias = ctx.saved_tensors
        desc = ctx.desc
        grad_out = grad_out.contiguous()
        L = _lib.lib()
        with torch.cuda.device(input.device):
            gx, goff, gw = torch.empty_like(input), torch.empty_like(offset), torch.empty_like(weight)
            gmask = None if alpha is None else torch.empty_like(alpha)
            gbias = None if bias is None else torch.empty_like(bias)
            ws, ws_bytes = _lib.workspace(_lib.OP_DEFORM_BWD, desc, input.device)
            ev = _new_event(torch.cuda.current_stream(input.device))
            if ctx.sample_cache is not None:
                ctx.sample_cache.bind()
            _lib.check(L.d2c_deform_conv3d_bwd_ev(
                ctypes.byref(desc), _lib.ptr(grad_out), _lib.ptr(input), _lib.ptr(offset), _lib.ptr(alpha),
                _lib.ptr(weight), _lib.ptr(gx), _lib.ptr(goff), _lib.ptr(gmask), _lib.ptr(gw), _lib.ptr(gbias),
                _lib.ptr(ws), ws_bytes, _lib.stream_of(input), ctypes.c_void_p(ev.cuda_event)), "deform_conv3d backward")
            _BackwardState.params_ready = ev
        return (gx, goff, gmask, gw, gbias) + (None,) * 12


def deform_conv3d(input, offset, alpha, weight, bias, stride_d, stride_h, stride_w, pad_d, pad_h, pad_w,
                  dilation_d, dilation_h, dilation_w, groups, offset_groups):
    """dconv_native._ops.deform_conv3d (csrc/ops/dconv3d.h:188-226)."""
    return _DeformConv3dFunction.apply(
        input, offset, alpha, weight, bias, int(stride_d), int(stride_h), int(stride_w), int(pad_d), int(pad_h),
        int(pad_w), int(dilation_d), int(dilation_h), int(dilation_w), int(groups), int(offset_groups),
        _will_differentiate(input, offset, alpha, weight, bias))


class _DynDilatedConv3dFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, size_map, alpha, weight, bias, mode, stride, padding, dilation, groups, offset_groups,
                differentiated):
        input, size_map, weight = input.contiguous(), size_map.contiguous(), weight.contiguous()
        alpha = None if alpha is None else alpha.contiguous()
        bias = None if bias is None else bias.contiguous()
        _sanity_check(input, size_map, alpha, weight, bias)
        _check_groups(input, weight, bias, groups)
        desc = _lib.make_desc(input, weight, stride, padding, dilation, groups, offset_groups)
        out_dims = _lib.output_dims(desc, "dyn_dilated_conv3d")
        K = weight.shape[2] * weight.shape[3] * weight.shape[4]
        if tuple(size_map.shape[1:]) != (_lib.FIELD_CHANNELS[mode],) + out_dims:
            raise RuntimeError(
                f"size_map must be [B, {_lib.FIELD_CHANNELS[mode]}, {out_dims}] for mode '{mode}', got {tuple(size_map.shape)}")
        if alpha is not None and tuple(alpha.shape[1:]) != (offset_groups * K,) + out_dims:
            raise RuntimeError(_lib.lib().d2c_status_string(-7).decode())
        L = _lib.lib()
        with torch.cuda.device(input.device):
            y = torch.empty((input.shape[0], weight.shape[0]) + out_dims, dtype=input.dtype, device=input.device)
            ws, ws_bytes = _lib.workspace(_lib.OP_DYNDIL_FWD, desc, input.device)
            cache = _lib.SampleCache.for_forward(desc, input.device, differentiated)
            _lib.check(L.d2c_dyn_dilated_conv3d_fwd(
                ctypes.byref(desc), _lib.FIELD_MODES[mode], _lib.ptr(input), _lib.ptr(size_map), _lib.ptr(alpha),
                _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(y), _lib.ptr(ws), ws_bytes, _lib.stream_of(input)),
                "dyn_dilated_conv3d forward")
        ctx.save_for_backward(input, size_map, alpha, weight, bias)
        ctx.desc, ctx.mode = desc, mode
        ctx.sample_cache = _lib.finish_forward_cache(cache)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        input, size_map, alpha, weight, bias = ctx.saved_tensors
        desc = ctx.desc
        grad_out = grad_out.contiguous()
        L = _lib.lib()
        with torch.cuda.device(input.device):
            gx, gs, gw = torch.empty_like(input), torch.empty_like(size_map), torch.empty_like(weight)
            gmask = None if alpha is None else torch.empty_like(alpha)
            gbias = None if bias is None else torch.empty_like(bias)
            ws, ws_bytes = _lib.workspace(_lib.OP_DYNDIL_BWD, desc, input.device)
            ev = _new_event(torch.cuda.current_stream(input.device))
            if ctx.sample_cache is not None:
                ctx.sample_cache.bind()
            _lib.check(L.d2c_dyn_dilated_conv3d_bwd_ev(
                ctypes.byref(desc), _lib.FIELD_MODES[ctx.mode], _lib.ptr(grad_out), _lib.ptr(input),
                _lib.ptr(size_map), _lib.ptr(alpha), _lib.ptr(weight), _lib.ptr(gx), _lib.ptr(gs), _lib.ptr(gmask),
                _lib.ptr(gw), _lib.ptr(gbias), _lib.ptr(ws), ws_bytes, _lib.stream_of(input),
                ctypes.c_void_p(ev.cuda_event)), "dyn_dilated_conv3d backward")
            _BackwardState.params_ready = ev
        return (gx, gs, gmask, gw, gbias) + (None,) * 7


def dyn_dilated_conv3d(input, size_map, alpha, weight, bias, mode, stride, padding, dilation, groups,
                       offset_groups):
    """Deformable conv3d whose offsets come from a dilation field (no counterpart in
    the reference's compiled module: there the field is expanded to 3*K offset
    channels by offsets_from_size_map, utils/grid.py:72-98, before deform_conv3d)."""
    return _DynDilatedConv3dFunction.apply(input, size_map, alpha, weight, bias, mode, tuple(stride),
                                           tuple(padding), tuple(dilation), int(groups), int(offset_groups),
                                           _will_differentiate(input, size_map, alpha, weight, bias))


class _DeformConv1dFunction(torch.autograd.Function):
    """DeformConv1dFunction of the reference (csrc/ops/dconv1d.h:69-156)."""

    @staticmethod
    def forward(ctx, input, offset, alpha, weight, bias, stride, padding, dilation, groups, offset_groups):
        input, offset, weight = input.contiguous(), offset.contiguous(), weight.contiguous()
        alpha = None if alpha is None else alpha.contiguous()
        bias = None if bias is None else bias.contiguous()
        for t, nd, name in ((input, 3, "input"), (offset, 3, "offset"), (alpha, 3, "alpha"), (weight, 3, "weight"),
                            (bias, 1, "bias")):
            if t is not None:
                _require(t.dim() == nd, f"{name}.ndimension() == {nd}")
                _require(t.is_cuda, f"{name}.device().is_cuda()")
                if t.dtype != input.dtype:
                    raise RuntimeError(f"expected scalar type {input.dtype} but found {t.dtype}")
        if input.dtype not in (torch.float32, torch.float64):
            raise RuntimeError(f'"deform_conv1d" not implemented for \'{input.dtype}\'')
        _check_groups(input, weight, bias, groups)
        K = weight.shape[2]
        # the [B, C, 1, 1, L] view of the problem
        desc = _lib.ConvDesc(_lib.dtype_code(input), input.shape[0], input.shape[1], weight.shape[0], 1, 1,
                             input.shape[2], 1, 1, K, 1, 1, stride, 0, 0, padding, 1, 1, dilation, groups,
                             offset_groups)
        Lo = _lib.output_dims(desc, "deform_conv1d")[2]
        if offset.shape[0] != input.shape[0] or offset.shape[1] != offset_groups * K or offset.shape[2] != Lo:
            raise RuntimeError(f"offset output dims do not match computed dims. Got: {tuple(offset.shape)} but expected: "
                               f"{(input.shape[0], offset_groups * K, Lo)}")
        if alpha is not None and tuple(alpha.shape) != tuple(offset.shape):
            raise RuntimeError(f"mask output dims do not match computed dims. Got: {tuple(alpha.shape)} but expected: "
                               f"{tuple(offset.shape)}")
        L = _lib.lib()
        with torch.cuda.device(input.device):
            y = torch.empty((input.shape[0], weight.shape[0], Lo), dtype=input.dtype, device=input.device)
            _lib.check(L.d2c_deform_conv1d_fwd(ctypes.byref(desc), _lib.ptr(input), _lib.ptr(offset), _lib.ptr(alpha),
                                               _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(y), _lib.stream_of(input)),
                       "deform_conv1d forward")
        ctx.save_for_backward(input, offset, alpha, weight, bias)
        ctx.desc = desc
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        input, offset, alpha, weight, bias = ctx.saved_tensors
        desc = ctx.desc
        grad_out = grad_out.contiguous()
        L = _lib.lib()
        with torch.cuda.device(input.device):
            gx, goff, gw = torch.empty_like(input), torch.empty_like(offset), torch.empty_like(weight)
            galpha = None if alpha is None else torch.empty_like(alpha)
            gbias = None if bias is None else torch.empty_like(bias)
            ws, ws_bytes = _lib.workspace(_lib.OP_DEFORM_BWD, desc, input.device)
            _lib.check(L.d2c_deform_conv1d_bwd(
                ctypes.byref(desc), _lib.ptr(grad_out), _lib.ptr(input), _lib.ptr(offset), _lib.ptr(alpha),
                _lib.ptr(weight), _lib.ptr(gx), _lib.ptr(goff), _lib.ptr(galpha), _lib.ptr(gw), _lib.ptr(gbias),
                _lib.ptr(ws), ws_bytes, _lib.stream_of(input)), "deform_conv1d backward")
        return (gx, goff, galpha, gw, gbias) + (None,) * 5


class _HeadConv3dFunction(torch.autograd.Function):
    """Deformable / dynamic-dilated conv3d that takes the predictor's RAW output: the split into geometry and mask
    channels and their activations (network/layers.py:107-120, 171-181, 302-313) happen inside the kernels, and
    the backward returns the gradient w.r.t. the raw tensor."""

    @staticmethod
    def forward(ctx, input, raw, weight, bias, field_mode, mask_channel0, mask_act, size_act, stride, padding,
                dilation, groups, offset_groups, differentiated):
        input, raw, weight = input.contiguous(), raw.contiguous(), weight.contiguous()
        bias = None if bias is None else bias.contiguous()
        for t, nd, name in ((input, 5, "input"), (raw, 5, "deformation"), (weight, 5, "weight"), (bias, 1, "bias")):
            if t is not None:
                _require(t.dim() == nd, f"{name}.ndimension() == {nd}")
                _require(t.is_cuda, f"{name}.device().is_cuda()")
                if t.dtype != input.dtype:
                    raise RuntimeError(f"expected scalar type {input.dtype} but found {t.dtype}")
        if input.dtype not in (torch.float32, torch.float64):
            raise RuntimeError(f'"deform_conv3d" not implemented for \'{input.dtype}\'')
        _require(raw.size(0) == input.size(0), "offset.size(0) == input.size(0)")
        _check_groups(input, weight, bias, groups)
        desc = _lib.make_desc(input, weight, stride, padding, dilation, groups, offset_groups)
        out_dims = _lib.output_dims(desc, "deform_conv3d")
        if tuple(raw.shape[2:]) != out_dims:
            raise RuntimeError(_lib.lib().d2c_status_string(-6).decode())
        head = _lib.HeadDesc(raw.shape[1], 0, mask_channel0, _lib.MASK_ACTS[mask_act], _lib.SIZE_ACTS[size_act])
        L = _lib.lib()
        fm = -1 if field_mode is None else _lib.FIELD_MODES[field_mode]
        op = _lib.OP_DEFORM_FWD if field_mode is None else _lib.OP_DYNDIL_FWD
        with torch.cuda.device(input.device):
            y = torch.empty((input.shape[0], weight.shape[0]) + out_dims, dtype=input.dtype, device=input.device)
            ws, ws_bytes = _lib.head_workspace(op, desc, head, max(fm, 0), input.device)
            args = (_lib.ptr(input), _lib.ptr(raw), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(y), _lib.ptr(ws), ws_bytes,
                    _lib.stream_of(input))
            cache = _lib.SampleCache.for_forward(desc, input.device, differentiated)
            if field_mode is None:
                rc = L.d2c_deform_conv3d_head_fwd(ctypes.byref(desc), ctypes.byref(head), *args)
            else:
                rc = L.d2c_dyn_dilated_conv3d_head_fwd(ctypes.byref(desc), ctypes.byref(head), fm, *args)
            _lib.check(rc, "deform_conv3d (fused head) forward")
        ctx.save_for_backward(input, raw, weight, bias)
        ctx.desc, ctx.head, ctx.fm = desc, head, fm
        ctx.sample_cache = _lib.finish_forward_cache(cache)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        input, raw, weight, bias = ctx.saved_tensors
        desc, head, fm = ctx.desc, ctx.head, ctx.fm
        grad_out = grad_out.contiguous()
        L = _lib.lib()
        op = _lib.OP_DEFORM_BWD if fm < 0 else _lib.OP_DYNDIL_BWD
        with torch.cuda.device(input.device):
            gx, graw, gw = torch.empty_like(input), torch.empty_like(raw), torch.empty_like(weight)
            gbias = None if bias is None else torch.empty_like(bias)
            ws, ws_bytes = _lib.head_workspace(op, desc, head, max(fm, 0), input.device)
            ev = _new_event(torch.cuda.current_stream(input.device))
            args = (_lib.ptr(grad_out), _lib.ptr(input), _lib.ptr(raw), _lib.ptr(weight), _lib.ptr(gx), _lib.ptr(graw),
                    _lib.ptr(gw), _lib.ptr(gbias), _lib.ptr(ws), ws_bytes, _lib.stream_of(input),
                    ctypes.c_void_p(ev.cuda_event))
            if ctx.sample_cache is not None:
                ctx.sample_cache.bind()
            if fm < 0:
                rc = L.d2c_deform_conv3d_head_bwd(ctypes.byref(desc), ctypes.byref(head), *args)
            else:
                rc = L.d2c_dyn_dilated_conv3d_head_bwd(ctypes.byref(desc), ctypes.byref(head), fm, *args)
            _lib.check(rc, "deform_conv3d (fused head) backward")
            _BackwardState.params_ready = ev
        return (gx, graw, gw, gbias) + (None,) * 10


def deform_conv3d_head(input, raw, weight, bias, field_mode, modulated, mask_act, size_act, stride, padding, dilation,
                       groups, offset_groups):
    """The layer's op on the predictor's raw output `raw` = [geometry channels | G*K mask logits (if modulated)]:
    geometry = 3*G*K offsets (field_mode None) or the 1..3 channels of a dilation field ("x", "xy", "xxz", "xyz").
    mask_act: "sigmoid" | "relu" | "tanh" | "linear" | "none"; size_act: "elu" | "relu" | "relu_plus_one" | "linear".
    No counterpart in the reference's compiled module, which is called after the split and the activations."""
    K = weight.shape[2] * weight.shape[3] * weight.shape[4]
    geo = 3 * offset_groups * K if field_mode is None else _lib.FIELD_CHANNELS[field_mode]
    want = geo + (offset_groups * K if modulated else 0)
    if raw.dim() != 5 or raw.shape[1] != want:
        raise RuntimeError(f"the deformation tensor must have {want} channels, got {tuple(raw.shape)}")
    return _HeadConv3dFunction.apply(input, raw, weight, bias, field_mode, geo if modulated else -1, mask_act,
                                     size_act if field_mode is not None else "linear", tuple(stride), tuple(padding),
                                     tuple(dilation), int(groups), int(offset_groups),
                                     _will_differentiate(input, raw, weight, bias))


def deform_conv1d(input, offset, alpha, weight, bias, stride, padding, dilation, groups, offset_groups):
    """dconv_native._ops.deform_conv1d (csrc/ops/dconv1d.h:158-186, dconv1d_gpu.cu): modulated deformable conv1d
    with one offset per (offset group, tap, output position) and linear interpolation, out-of-range neighbours
    read as 0.  Forward, grad_input, grad_weight and grad_bias run on the library's generic kernels over the
    [B, C, 1, 1, L] view of the problem; grad_offset / grad_alpha come from a kernel of their own that follows the
    1-D reference's rule at integer sampling positions (`x0 -= 1`, dconv1d_gpu.cu:334-337)."""
    one = lambda v: int(v[0]) if isinstance(v, (tuple, list)) else int(v)
    return _DeformConv1dFunction.apply(input, offset, alpha, weight, bias, one(stride), one(padding), one(dilation),
                                       int(groups), int(offset_groups))


def corners(input_shape, weight_shape, offset, stride, padding, dilation, offset_groups):
    """Integer floor corners [B, G*K, 3, V] the kernels derive from `offset`."""
    offset = offset.contiguous()
    desc = _lib.ConvDesc(_lib.dtype_code(offset), input_shape[0], input_shape[1], weight_shape[0],
                         input_shape[2], input_shape[3], input_shape[4], weight_shape[2], weight_shape[3],
                         weight_shape[4], *stride, *padding, *dilation, 1, offset_groups)
    V = 1
    for d in _lib.output_dims(desc):
        V *= d
    K = weight_shape[2] * weight_shape[3] * weight_shape[4]
    out = torch.empty((input_shape[0], offset_groups * K, 3, V), dtype=torch.int32, device=offset.device)
    with torch.cuda.device(offset.device):
        _lib.check(_lib.lib().d2c_deform_conv3d_corners(ctypes.byref(desc), _lib.ptr(offset), _lib.ptr(out),
                                                        _lib.stream_of(offset)), "corners")
    return out


def field_corners(input_shape, weight_shape, size_map, mode, stride, padding, dilation, offset_groups):
    size_map = size_map.contiguous()
    desc = _lib.ConvDesc(_lib.dtype_code(size_map), input_shape[0], input_shape[1], weight_shape[0],
                         input_shape[2], input_shape[3], input_shape[4], weight_shape[2], weight_shape[3],
                         weight_shape[4], *stride, *padding, *dilation, 1, offset_groups)
    V = 1
    for d in _lib.output_dims(desc):
        V *= d
    K = weight_shape[2] * weight_shape[3] * weight_shape[4]
    out = torch.empty((input_shape[0], offset_groups * K, 3, V), dtype=torch.int32, device=size_map.device)
    with torch.cuda.device(size_map.device):
        _lib.check(_lib.lib().d2c_dyn_dilated_conv3d_corners(
            ctypes.byref(desc), _lib.FIELD_MODES[mode], _lib.ptr(size_map), _lib.ptr(out),
            _lib.stream_of(size_map)), "field corners")
    return out


def _get_max_intermediate_elements():
    return int(_lib.lib().d2c_get_max_intermediate_elements())


def _set_max_intermediate_elements(n):
    _lib.lib().d2c_set_max_intermediate_elements(int(n))


# dconv_native._ops.config (csrc/ops/dconv.cpp:9-11)
config = types.SimpleNamespace(
    get_max_intermediate_elements=_get_max_intermediate_elements,
    set_max_intermediate_elements=_set_max_intermediate_elements,
)
