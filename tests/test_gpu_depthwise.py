"""GPU parity tests of the depthwise conv3d kernels (through the C ABI) against the CPU
oracle, following ops/fast-depthwise-conv3d/test/test_conv3d_depthwise.py:25-96:
stride x dilation in {1,2}^2, channel multiplier {1,2}, float/double/half with
atol 1e-5 / 1e-5 / 1e-2."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

ATOL = {torch.float32: 1e-5, torch.float64: 1e-5, torch.float16: 1e-2}


@pytest.fixture(scope="module")
def dw():
    from d2conv3d_b200 import _lib, fast_depthwise_conv3d
    _lib.lib()
    return fast_depthwise_conv3d


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.float16])
@pytest.mark.parametrize("stride,dilation", [(1, 1), (2, 1), (1, 2), (2, 2)])
@pytest.mark.parametrize("mult,bias", [(1, True), (2, False)])
def test_depthwise_vs_oracle(dw, dtype, stride, dilation, mult, bias):
    torch.manual_seed(0)
    pad = dilation
    m = dw.DepthwiseConv3d(2, 2 * mult, kernel_size=3, bias=bias, stride=stride, padding=pad, dilation=dilation).to("cuda", dtype)
    x = torch.randn(2, 2, 6, 6, 6, device="cuda", dtype=dtype).div_(2).requires_grad_()
    y = m(x)
    gy = torch.randn_like(y) / 2
    y.backward(gy)
    np64 = lambda t: t.detach().double().cpu().numpy()
    wy = orc.depthwise_conv3d_fwd(np64(x), np64(m.weight), np64(m.bias) if bias else None, stride, pad, dilation)
    wgx, wgw, wgb = orc.depthwise_conv3d_bwd(np64(gy), np64(x), np64(m.weight), bias, stride, pad, dilation)
    atol = ATOL[dtype]
    assert y.dtype == dtype
    assert np.abs(np64(y) - wy).max() <= atol
    assert np.abs(np64(x.grad) - wgx).max() <= atol
    assert np.abs(np64(m.weight.grad) - wgw).max() <= atol * (10 if dtype == torch.float16 else 1)
    if bias:
        assert np.abs(np64(m.bias.grad) - wgb).max() <= atol * (10 if dtype == torch.float16 else 1)


def test_depthwise_other_kernel_shapes_and_larger_tile(dw):
    torch.manual_seed(1)
    for k, pad in (((1, 3, 3), (0, 1, 1)), ((3, 5, 3), (1, 2, 1)), (3, 1)):
        m = dw.DepthwiseConv3d(5, 5, kernel_size=k, padding=pad).to("cuda", torch.float32)
        x = torch.randn(3, 5, 4, 9, 13, device="cuda").requires_grad_()
        y = m(x)
        gy = torch.randn_like(y)
        y.backward(gy)
        np32 = lambda t: t.detach().cpu().numpy()
        wy = orc.depthwise_conv3d_fwd(np32(x), np32(m.weight), np32(m.bias), 1, pad, 1)
        wgx, wgw, wgb = orc.depthwise_conv3d_bwd(np32(gy), np32(x), np32(m.weight), True, 1, pad, 1)
        assert np.abs(np32(y) - wy).max() <= 1e-5
        assert np.abs(np32(x.grad) - wgx).max() <= 1e-5
        assert np.abs(np32(m.weight.grad) - wgw).max() <= 1e-4 * max(1.0, np.abs(wgw).max())
        assert np.abs(np32(m.bias.grad) - wgb).max() <= 1e-4 * max(1.0, np.abs(wgb).max())


@pytest.mark.parametrize("shape,dtype,misalign", [
    ((2, 8, 4, 6, 8), torch.float32, False),      # planes staged by bulk copies, one volume per chunk
    ((2, 640, 2, 4, 8), torch.float32, False),    # small volumes: two per chunk
    ((2, 640, 2, 4, 8), torch.float16, False),    # half: 64-byte planes
    ((2, 8, 5, 6, 8), torch.float32, False),      # depth not a multiple of the march's unroll
    ((2, 64, 2, 5, 7), torch.float32, False),     # 140-byte planes cannot be bulk-copied: register-window march
    ((1, 3, 3, 5, 7), torch.float32, False),      # odd everything
    ((1, 2, 8, 56, 56), torch.float32, False),    # forward fits shared memory with one block per SM, weight gradient does not
    ((2, 8, 4, 6, 8), torch.float32, True),       # tensors at a 4-byte offset: no bulk copy possible
    ((1, 4, 1, 9, 32), torch.float64, False),     # single plane, double, odd height
    # fp32 with even W: packed-FMA kernels (4-row x 2-column patches forward, 2 x 2 for the weight gradient)
    ((1, 4, 1, 10, 8), torch.float32, False),     # one plane; H = 10 leaves a 2-row patch at the bottom
    ((2, 3, 2, 7, 6), torch.float32, False),      # two planes, odd H (7 = 4 + 3 rows), W % 4 == 2
    ((1, 5, 3, 30, 54), torch.float32, False),    # the benchmark's plane size, depth 3 (one full rotation)
    ((3, 2, 7, 5, 12), torch.float32, False),     # depth 7, H = 5 (patch of one valid row), W % 4 == 0
    ((2, 300, 4, 2, 4), torch.float32, False),    # tiny volumes, several per chunk, H smaller than a patch
])
def test_depthwise_3x3x3_fast_paths(dw, shape, dtype, misalign):
    """The 3x3x3 / stride 1 / padding 1 case has three implementations chosen by size and alignment
    (bulk-copy pipeline, register-window march, generic); every one must match the oracle."""
    from d2conv3d_b200 import _lib
    torch.manual_seed(11)
    B, C = shape[:2]

    def make(*sh):
        n = int(np.prod(sh))
        if misalign:
            return torch.randn(n + 1, device="cuda", dtype=dtype)[1:].view(*sh)
        return torch.randn(*sh, device="cuda", dtype=dtype)

    x = make(*shape).div_(2).requires_grad_()
    w = (torch.randn(C, 1, 3, 3, 3, device="cuda", dtype=dtype) / 4).requires_grad_()
    b = torch.randn(C, device="cuda", dtype=dtype).requires_grad_()
    y = dw._ops.depthwise_separable_conv3d(x, w, b, 1, 1, 1)
    gy = make(*shape).div_(2)
    y.backward(gy)
    np64 = lambda t: t.detach().double().cpu().numpy()
    wy = orc.depthwise_conv3d_fwd(np64(x), np64(w), np64(b), 1, 1, 1)
    wgx, wgw, wgb = orc.depthwise_conv3d_bwd(np64(gy), np64(x), np64(w), True, 1, 1, 1)
    atol = ATOL[dtype]
    assert np.abs(np64(y) - wy).max() <= atol
    assert np.abs(np64(x.grad) - wgx).max() <= atol
    scale = max(1.0, float(np.abs(wgw).max()))
    assert np.abs(np64(w.grad) - wgw).max() <= (1e-2 if dtype == torch.float16 else 1e-4) * scale
    _lib.device_status()


def test_non_finite_input_next_to_a_border_stays_local(dw):
    """The packed-FMA kernels read a neighbouring row's element where a patch touches the left / right border
    and must discard it (not multiply it by zero): an Inf in the last column of a row may only reach the outputs
    cuDNN lets it reach."""
    torch.manual_seed(5)
    x = torch.randn(1, 2, 3, 6, 8, device="cuda")
    x[0, 0, 1, 2, 7] = float("inf")       # last column of row 2: precedes column 0 of row 3 in memory
    x[0, 1, 1, 3, 0] = float("inf")       # first column of row 3: follows the last column of row 2
    w = torch.randn(2, 1, 3, 3, 3, device="cuda").abs() + 0.1      # positive weights: Inf, never Inf - Inf
    y = dw._ops.depthwise_separable_conv3d(x, w, None, 1, 1, 1)
    ref = torch.nn.functional.conv3d(x, w, None, padding=1, groups=2)
    assert torch.equal(torch.isfinite(y), torch.isfinite(ref))
    fin = torch.isfinite(ref)
    assert torch.allclose(y[fin], ref[fin], atol=1e-5)


def test_autocast_keeps_half(dw):
    inp = torch.randn(2, 2, 5, 5, 5).to(dtype=torch.half, device="cuda")
    conv = dw.DepthwiseConv3d(2, 2, kernel_size=3).cuda()
    with torch.autocast("cuda"):
        assert conv(inp).dtype == torch.half


def test_padding_mode_replicate(dw):
    torch.manual_seed(3)
    conv = dw.DepthwiseConv3d(3, 3, kernel_size=3, padding=1, padding_mode="replicate").cuda()
    ref = torch.nn.Conv3d(3, 3, 3, padding=1, padding_mode="replicate", groups=3).cuda()
    ref.load_state_dict(conv.state_dict())
    x = torch.randn(2, 3, 4, 5, 6, device="cuda")
    xp = torch.nn.functional.pad(x, (1, 1, 1, 1, 1, 1), mode="replicate")
    want = orc.depthwise_conv3d_fwd(xp.cpu().numpy(), conv.weight.detach().cpu().numpy(), conv.bias.detach().cpu().numpy())
    assert np.abs(conv(x).detach().cpu().numpy() - want).max() <= 1e-5
