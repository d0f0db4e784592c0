"""A bounded device-side wait that runs out: the kernel returns, the status word is raised, the host sees
D2C_ERR_DEVICE_TIMEOUT exactly once, and the context keeps working.

The wait is made to run out on purpose in the harmless form: a one-warp kernel waits about a millisecond on a
barrier that nothing arrives on (no memory access, no trap, no endless loop), then returns normally."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TIMEOUT = 2     # D2C_ERR_DEVICE_TIMEOUT


def test_wait_expiry_is_reported_once_and_the_context_survives():
    from d2conv3d_b200 import _lib, fast_depthwise_conv3d
    L = _lib.lib()
    _lib.device_status()                                    # healthy to begin with
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.d2c_selftest_wait_expiry(1000, stream) == 0    # ~1 ms budget
    assert L.d2c_device_status() == TIMEOUT
    assert L.d2c_device_status() == 0                       # reported once, then cleared
    # the kernel returned normally: the same context runs ordinary work afterwards
    x = torch.randn(1, 4, 3, 5, 6, device="cuda")
    w = torch.randn(4, 1, 3, 3, 3, device="cuda")
    y = fast_depthwise_conv3d._ops.depthwise_separable_conv3d(x, w, None, 1, 1, 1)
    want = torch.nn.functional.conv3d(x, w, None, 1, 1, 1, 4)
    assert float((y - want).abs().max()) <= 1e-5
    _lib.device_status()


def test_next_library_call_reports_a_pending_timeout_without_launching():
    from d2conv3d_b200 import _lib
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.d2c_selftest_wait_expiry(500, stream) == 0
    torch.cuda.synchronize()
    assert L.d2c_device_status_peek() == TIMEOUT            # peek neither clears ...
    assert L.d2c_device_status_peek() == TIMEOUT
    x = torch.randn(1, 4, 3, 5, 6, device="cuda")
    w = torch.randn(4, 1, 3, 3, 3, device="cuda")
    y = torch.full_like(x, 7.0)
    desc = _lib.make_desc(x, w, (1, 1, 1), (1, 1, 1), (1, 1, 1), 4, 1)
    n0 = _lib.launch_count()
    rc = L.d2c_depthwise_conv3d_fwd(ctypes.byref(desc), _lib.ptr(x), _lib.ptr(w), None, _lib.ptr(y), stream)
    assert rc == TIMEOUT and _lib.launch_count() == n0      # ... the next compute call does, launching nothing
    torch.cuda.synchronize()
    assert bool((y == 7.0).all())
    assert L.d2c_depthwise_conv3d_fwd(ctypes.byref(desc), _lib.ptr(x), _lib.ptr(w), None, _lib.ptr(y), stream) == 0
    _lib.device_status()


def test_invalid_budget_is_rejected():
    from d2conv3d_b200 import _lib
    L = _lib.lib()
    assert L.d2c_selftest_wait_expiry(0, None) == -3
    assert L.d2c_selftest_wait_expiry(10 ** 6, None) == -3
