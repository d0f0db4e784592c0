"""GPU test of d2c_depthwise_conv3d_bwd_noalloc -- the depthwise backward for callers that cannot
allocate device memory (a process with a fixed, pre-planned device-memory budget, or a loop that must
never hit the device-wide synchronisation of cudaMalloc/cudaFree).  Its weight-gradient accumulators
live in a fixed array inside the library instead of a caller-supplied workspace.

The entry point is called through the C ABI and compared with the workspace-taking entry point
(d2c_depthwise_conv3d_bwd) on the same inputs, twice in a row with different data: the second call
finds the first call's sums still in the shared array and must not be affected by them.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

ATOL = 1e-5   # the bound the depthwise tests use for float32


def _call_pair(L, _lib, desc, gy, x, w):
    """-> ((gx, gw, gb) from the workspace entry point, (gx, gw, gb) from the no-alloc entry point)"""
    stream = _lib.stream_of(x)
    ref = [torch.empty_like(x), torch.empty_like(w), torch.empty(w.shape[0], device=x.device, dtype=x.dtype)]
    ws, ws_bytes = _lib.workspace(_lib.OP_DW_BWD, desc, x.device)
    _lib.check(L.d2c_depthwise_conv3d_bwd(ctypes.byref(desc), _lib.ptr(gy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(ref[0]),
                                          _lib.ptr(ref[1]), _lib.ptr(ref[2]), _lib.ptr(ws), ws_bytes, stream), "bwd")
    got = [torch.full_like(t, float("nan")) for t in ref]
    _lib.check(L.d2c_depthwise_conv3d_bwd_noalloc(ctypes.byref(desc), _lib.ptr(gy), _lib.ptr(x), _lib.ptr(w),
                                                  _lib.ptr(got[0]), _lib.ptr(got[1]), _lib.ptr(got[2]), stream),
               "bwd_noalloc")
    torch.cuda.synchronize()
    return ref, got


def _torch_grads(gy, x, w, groups):
    """The same three gradients from PyTorch's own grouped conv3d (cuDNN / native kernels)."""
    xr, wr = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    y = torch.nn.functional.conv3d(xr, wr, None, 1, 1, 1, groups)
    y.backward(gy)
    return [xr.grad, wr.grad, gy.sum(dim=(0, 2, 3, 4))]


# (channels, channel multiplier, clip dims): multiplier 2 with odd sizes runs the generic weight-gradient kernel;
# multiplier 1 with an even width and 16-byte-aligned planes runs the packed-FMA 3x3x3 kernels, whose per-warp
# flushes accumulate into the same built-in array
SHAPES = [(24, 2, (5, 9, 11)), (16, 1, (6, 6, 12)), (8, 1, (4, 7, 9))]


@pytest.mark.parametrize("C,mult,dims", SHAPES)
def test_noalloc_depthwise_backward_matches_workspace_version_twice(C, mult, dims):
    from d2conv3d_b200 import _lib
    L = _lib.lib()
    assert torch.cuda.is_available()
    torch.manual_seed(11)
    for call in range(2):
        x = torch.randn(3, C, *dims, device="cuda") * (1.0 + call)
        w = torch.randn(C * mult, 1, 3, 3, 3, device="cuda")
        desc = _lib.make_desc(x, w, (1, 1, 1), (1, 1, 1), (1, 1, 1), C, 1)
        od = _lib.output_dims(desc)
        gy = torch.randn(3, C * mult, *od, device="cuda") * (0.5 + 3.0 * call)
        ref, got = _call_pair(L, _lib, desc, gy, x, w)
        want = _torch_grads(gy, x, w, C)
        for name, a, b, t in zip(("grad_x", "grad_w", "grad_bias"), ref, got, want):
            assert torch.isfinite(b).all(), f"call {call}: {name} not fully written"
            scale = max(1.0, float(a.abs().max()))
            assert float((a - b).abs().max()) <= ATOL * scale, f"call {call}: {name} vs the workspace entry point"
            assert float((t - b).abs().max()) <= 1e-4 * scale, f"call {call}: {name} vs torch conv3d"


def test_noalloc_call_leaves_device_memory_untouched():
    """Neither the driver's free-memory figure nor PyTorch's allocator statistics move across the call
    (set-up of the built-in array's address happened in an earlier call on this device)."""
    from d2conv3d_b200 import _lib
    L = _lib.lib()
    C = 16
    x = torch.randn(2, C, 6, 6, 12, device="cuda")
    w = torch.randn(C, 1, 3, 3, 3, device="cuda")
    gy = torch.randn(2, C, 6, 6, 12, device="cuda")
    desc = _lib.make_desc(x, w, (1, 1, 1), (1, 1, 1), (1, 1, 1), C, 1)
    out = [torch.empty_like(x), torch.empty_like(w), torch.empty(C, device="cuda")]
    args = (ctypes.byref(desc), _lib.ptr(gy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(out[0]), _lib.ptr(out[1]),
            _lib.ptr(out[2]), _lib.stream_of(x))
    _lib.check(L.d2c_depthwise_conv3d_bwd_noalloc(*args), "first call (does the one-time set-up)")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    stats0 = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    _lib.check(L.d2c_depthwise_conv3d_bwd_noalloc(*args), "second call")
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 >= free0, f"device free memory dropped by {free0 - free1} bytes across the call"
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == stats0


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    from d2conv3d_b200 import _lib
    L = _lib.lib()
    C = 1280                                   # 1280 * 27 = 34560 accumulator slots > 32768
    x = torch.zeros(1, C, 1, 2, 2, device="cuda")
    w = torch.zeros(C, 1, 3, 3, 3, device="cuda")
    desc = _lib.make_desc(x, w, (1, 1, 1), (1, 1, 1), (1, 1, 1), C, 1)
    gy = torch.zeros(1, C, 1, 2, 2, device="cuda")
    gx, gw = torch.empty_like(x), torch.empty_like(w)
    rc = L.d2c_depthwise_conv3d_bwd_noalloc(ctypes.byref(desc), _lib.ptr(gy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(gx),
                                            _lib.ptr(gw), None, _lib.stream_of(x))
    assert rc == -12
    assert b"32768" in L.d2c_status_string(rc)
    # without a weight gradient no scratch is needed, so the same shape is accepted
    rc = L.d2c_depthwise_conv3d_bwd_noalloc(ctypes.byref(desc), _lib.ptr(gy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(gx),
                                            None, None, _lib.stream_of(x))
    assert rc == 0
    torch.cuda.synchronize()
