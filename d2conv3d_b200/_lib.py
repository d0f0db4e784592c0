"""ctypes binding of libd2conv3d.so (the C ABI declared in include/d2conv3d.h).

PyTorch is used only for device memory and the current stream: every call passes
raw device pointers, sizes and a cudaStream_t across the C boundary.  There is no
CPU or PyTorch fallback -- if the library is missing or a call fails, an error is
raised.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libd2conv3d.so")

F32, F64, F16 = 0, 1, 2
MATH_MODES = {"auto": 0, "fp32": 1, "bf16x3": 2, "bf16": 3}
FIELD_MODES = {"x": 0, "xy": 1, "xxz": 2, "xyz": 3}
FIELD_CHANNELS = {"x": 1, "xy": 2, "xxz": 2, "xyz": 3}
OP_DEFORM_FWD, OP_DEFORM_BWD, OP_DYNDIL_FWD, OP_DYNDIL_BWD, OP_DW_FWD, OP_DW_BWD = range(6)

_DTYPES = {torch.float32: F32, torch.float64: F64, torch.float16: F16}


class ConvDesc(ctypes.Structure):
    """d2c_conv_desc"""

    _fields_ = [(n, ctypes.c_int32) for n in (
        "dtype", "batch", "in_channels", "out_channels", "in_d", "in_h", "in_w",
        "kd", "kh", "kw", "stride_d", "stride_h", "stride_w", "pad_d", "pad_h", "pad_w",
        "dil_d", "dil_h", "dil_w", "groups", "offset_groups")]


class HeadDesc(ctypes.Structure):
    """d2c_head_desc"""

    _fields_ = [(n, ctypes.c_int32) for n in ("raw_channels", "geo_channel0", "mask_channel0", "mask_act", "size_act")]


MASK_ACTS = {"linear": 0, "none": 0, "sigmoid": 1, "relu": 2, "tanh": 3}
SIZE_ACTS = {"linear": 0, "elu": 1, "relu": 2, "relu_plus_one": 3}


class SampleCacheStruct(ctypes.Structure):
    """d2c_sample_cache"""

    _fields_ = [("data", ctypes.c_void_p), ("bytes", ctypes.c_size_t), ("format", ctypes.c_int32),
                ("reserved", ctypes.c_int32)]


class ProfileRecord(ctypes.Structure):
    """d2c_profile_record"""

    _fields_ = [("name", ctypes.c_char_p), ("ms", ctypes.c_float)]


_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m d2conv3d_b200.build` "
                "(there is no fallback implementation)")
        L = ctypes.CDLL(LIB_PATH)
        vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        dp = ctypes.POINTER(ConvDesc)
        L.d2c_output_dims.argtypes = [dp, ctypes.POINTER(ctypes.c_int32)]
        L.d2c_deform_conv3d_check.argtypes = [dp, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
        L.d2c_workspace_bytes.argtypes = [i32, dp]
        L.d2c_workspace_bytes.restype = sz
        L.d2c_status_string.argtypes = [i32]
        L.d2c_status_string.restype = ctypes.c_char_p
        L.d2c_last_cuda_error.restype = ctypes.c_char_p
        L.d2c_launch_count.restype = ctypes.c_uint64
        L.d2c_device_status_clear.restype = None
        L.d2c_selftest_wait_expiry.argtypes = [ctypes.c_uint32, vp]
        L.d2c_profile_enable.argtypes = [i32]
        L.d2c_profile_read.argtypes = [ctypes.POINTER(ProfileRecord), i32, ctypes.POINTER(i32)]
        L.d2c_set_math_mode.argtypes = [i32]
        L.d2c_get_max_intermediate_elements.restype = ctypes.c_uint64
        L.d2c_set_max_intermediate_elements.argtypes = [ctypes.c_uint64]
        L.d2c_set_max_intermediate_elements.restype = None
        L.d2c_sample_cache_bytes.argtypes = [dp]
        L.d2c_sample_cache_bytes.restype = sz
        L.d2c_bind_sample_cache.argtypes = [ctypes.POINTER(SampleCacheStruct)]
        L.d2c_deform_conv3d_fwd.argtypes = [dp] + [vp] * 7 + [sz, vp]
        L.d2c_deform_conv3d_bwd.argtypes = [dp] + [vp] * 11 + [sz, vp]
        L.d2c_deform_conv3d_bwd_ev.argtypes = [dp] + [vp] * 11 + [sz, vp, vp]
        L.d2c_dyn_dilated_conv3d_bwd_ev.argtypes = [dp, i32] + [vp] * 11 + [sz, vp, vp]
        L.d2c_deform_conv3d_corners.argtypes = [dp, vp, vp, vp]
        L.d2c_deform_conv1d_fwd.argtypes = [dp] + [vp] * 6 + [vp]
        L.d2c_deform_conv1d_bwd.argtypes = [dp] + [vp] * 11 + [sz, vp]
        L.d2c_dyn_dilated_conv3d_fwd.argtypes = [dp, i32] + [vp] * 7 + [sz, vp]
        L.d2c_dyn_dilated_conv3d_bwd.argtypes = [dp, i32] + [vp] * 11 + [sz, vp]
        L.d2c_dyn_dilated_conv3d_corners.argtypes = [dp, i32, vp, vp, vp]
        hp = ctypes.POINTER(HeadDesc)
        L.d2c_head_workspace_bytes.argtypes = [i32, dp, hp, i32]
        L.d2c_head_workspace_bytes.restype = sz
        L.d2c_deform_conv3d_head_fwd.argtypes = [dp, hp] + [vp] * 6 + [sz, vp]
        L.d2c_deform_conv3d_head_bwd.argtypes = [dp, hp] + [vp] * 9 + [sz, vp, vp]
        L.d2c_dyn_dilated_conv3d_head_fwd.argtypes = [dp, hp, i32] + [vp] * 6 + [sz, vp]
        L.d2c_dyn_dilated_conv3d_head_bwd.argtypes = [dp, hp, i32] + [vp] * 9 + [sz, vp, vp]
        L.d2c_act_group_norm_workspace_bytes.argtypes = [i32, i32]
        L.d2c_act_group_norm_workspace_bytes.restype = sz
        L.d2c_act_group_norm_fwd.argtypes = [vp, vp, vp, vp, i32, i32, ctypes.c_longlong, i32, ctypes.c_float, i32,
                                             vp, sz, vp]
        L.d2c_act_group_norm_bwd_workspace_bytes.argtypes = [i32, i32, i32]
        L.d2c_act_group_norm_bwd_workspace_bytes.restype = sz
        L.d2c_act_group_norm_bwd.argtypes = [vp] * 7 + [i32, i32, ctypes.c_longlong, i32, ctypes.c_float, i32, vp, sz, vp]
        L.d2c_depthwise_conv3d_fwd.argtypes = [dp] + [vp] * 4 + [vp]
        L.d2c_depthwise_conv3d_bwd.argtypes = [dp] + [vp] * 7 + [sz, vp]
        L.d2c_depthwise_conv3d_bwd_noalloc.argtypes = [dp] + [vp] * 6 + [vp]
        _lib = L
    return _lib


def check(status, what):
    if status == 0:
        return
    L = lib()
    msg = L.d2c_status_string(status).decode()
    if status > 0:
        msg += ": " + L.d2c_last_cuda_error().decode()
    raise RuntimeError(f"{what}: {msg} (status {status})")


def dtype_code(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {t.dtype}") from None


def make_desc(x, w, stride, padding, dilation, groups, offset_groups):
    return ConvDesc(dtype_code(x), x.shape[0], x.shape[1], w.shape[0], x.shape[2], x.shape[3], x.shape[4],
                    w.shape[2], w.shape[3], w.shape[4], stride[0], stride[1], stride[2],
                    padding[0], padding[1], padding[2], dilation[0], dilation[1], dilation[2],
                    groups, offset_groups)


def output_dims(desc, what="conv3d"):
    out = (ctypes.c_int32 * 3)()
    check(lib().d2c_output_dims(ctypes.byref(desc), out), what)
    return tuple(out)


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_of(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def workspace(op, desc, device):
    n = lib().d2c_workspace_bytes(op, ctypes.byref(desc))
    if n == 0:
        return None, 0
    ws = torch.empty(n, dtype=torch.uint8, device=device)
    return ws, n


def head_workspace(op, desc, head, field_mode, device):
    n = lib().d2c_head_workspace_bytes(op, ctypes.byref(desc), ctypes.byref(head), field_mode)
    if n == 0:
        return None, 0
    return torch.empty(n, dtype=torch.uint8, device=device), n


_keep_samples = True


def set_keep_samples(on):
    """Whether a forward that will be differentiated keeps its blended samples (16-bit, B*Cin*K*V elements) for the
    weight gradient of its backward -- the reference computes them twice.  On by default; switch it off to trade the
    backward's speed for that memory.  Shapes above the intermediate-element cap never keep them."""
    global _keep_samples
    _keep_samples = bool(on)


def get_keep_samples():
    return _keep_samples


class SampleCache:
    """Buffer + descriptor handed from a forward call to its backward (d2c_sample_cache)."""

    def __init__(self, desc, device):
        n = lib().d2c_sample_cache_bytes(ctypes.byref(desc))
        self.buf = torch.empty(n, dtype=torch.uint8, device=device) if n else None
        self.c = SampleCacheStruct(self.buf.data_ptr() if n else None, n, 0, 0)

    @staticmethod
    def for_forward(desc, device, differentiated):
        """A bound cache for the forward call that follows, or None (nothing to keep / switched off)."""
        if not (differentiated and _keep_samples):
            return None
        cache = SampleCache(desc, device)
        if cache.buf is None:
            return None
        cache.bind()
        return cache

    def bind(self):
        """Applies to the next deformable forward / backward call of this thread."""
        check(lib().d2c_bind_sample_cache(ctypes.byref(self.c)), "bind_sample_cache")

    @property
    def kept(self):
        return self.c.format != 0


def finish_forward_cache(cache):
    """After the forward call: the cache if the kernels filled it, else None (buffer released)."""
    return cache if cache is not None and cache.kept else None


def set_math_mode(mode):
    """'auto' | 'fp32' | 'bf16x3' | 'bf16' -- how the Cin*K x Cout contraction is evaluated."""
    check(lib().d2c_set_math_mode(MATH_MODES[mode]), "set_math_mode")


def get_math_mode():
    code = lib().d2c_get_math_mode()
    return {v: k for k, v in MATH_MODES.items()}[code]


def device_status():
    """Synchronises, then raises (once: the report clears the flag) if a kernel's bounded wait gave up
    since the last report on this device."""
    check(lib().d2c_device_status(), "device status")


def device_status_clear():
    lib().d2c_device_status_clear()


def launch_count():
    """Kernels launched by the library in this process so far."""
    return int(lib().d2c_launch_count())


def profile_enable(on=True):
    check(lib().d2c_profile_enable(1 if on else 0), "profile_enable")


def profile_read(max_records=65536):
    """[(phase name, milliseconds)] since the last read; synchronises with the device."""
    recs = (ProfileRecord * max_records)()
    n = ctypes.c_int(0)
    check(lib().d2c_profile_read(recs, max_records, ctypes.byref(n)), "profile_read")
    return [(recs[i].name.decode(), float(recs[i].ms)) for i in range(n.value)]


class _ActGroupNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, groups, eps, relu):
        if not (x.is_cuda and x.dtype == torch.float32):
            raise RuntimeError("act_group_norm expects an fp32 CUDA tensor")
        x = x.contiguous()
        B, C = x.shape[0], x.shape[1]
        spatial = x.numel() // (B * C)
        L = lib()
        with torch.cuda.device(x.device):
            y = torch.empty_like(x)
            n = L.d2c_act_group_norm_workspace_bytes(B, groups)
            stats = torch.empty(n, dtype=torch.uint8, device=x.device)
            check(L.d2c_act_group_norm_fwd(ptr(x), ptr(weight), ptr(bias), ptr(y), B, C, spatial, groups, float(eps),
                                           1 if relu else 0, ptr(stats), n, stream_of(x)), "act_group_norm")
        ctx.save_for_backward(x, weight, stats)
        ctx.cfg = (B, C, spatial, groups, float(eps), 1 if relu else 0, bias is not None)
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy):
        x, weight, stats = ctx.saved_tensors
        B, C, spatial, groups, eps, relu, has_bias = ctx.cfg
        gy = gy.contiguous()
        L = lib()
        with torch.cuda.device(x.device):
            gx = torch.empty_like(x)
            gw = torch.empty(C, dtype=torch.float32, device=x.device) if weight is not None else None
            gb = torch.empty(C, dtype=torch.float32, device=x.device) if has_bias else None
            n = L.d2c_act_group_norm_bwd_workspace_bytes(B, C, groups)
            ws = torch.empty(n, dtype=torch.uint8, device=x.device)
            check(L.d2c_act_group_norm_bwd(ptr(x), ptr(weight), ptr(gy), ptr(stats), ptr(gx), ptr(gw), ptr(gb), B, C,
                                           spatial, groups, eps, relu, ptr(ws), n, stream_of(x)), "act_group_norm backward")
        return gx, gw, gb, None, None, None


def act_group_norm(x, weight, bias, groups, eps=1e-5, relu=True):
    """y = GroupNorm(relu(x)) for an fp32 CUDA tensor [B, C, *spatial]; differentiable in x, weight, bias."""
    return _ActGroupNorm.apply(x, weight, bias, int(groups), float(eps), bool(relu))
