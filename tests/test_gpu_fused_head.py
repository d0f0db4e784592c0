"""The deformation head fused into the op: the layers hand the predictor's raw output to the kernels, which split
it, activate the mask logits (sigmoid / relu / tanh / none) and the dilation field (elu+1 / relu / relu_plus_one /
linear) where they read them, and return the gradient w.r.t. the raw tensor.  Checked against the same layer with
`fused_head=False` (the reference's sequence: split, activations, op -- network/layers.py:107-120, 171-181,
302-313): output and every gradient (input, predictor weight and bias, layer weight and bias), tensor-core tier
(fp32, `auto` mode) and CUDA-core tier (fp64), and the kernel list of a forward pass: no activation or copy kernel
between the predictor convolution and this library's kernels."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def mods():
    import d2conv3d_b200
    from d2conv3d_b200 import _lib
    from d2conv3d_b200.dconv_native import modules
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    d2conv3d_b200.set_math_mode("auto")
    yield modules
    d2conv3d_b200.set_math_mode("auto")
    _lib.device_status()


def make_pair(modules, cls, cin, cout, dtype, **kw):
    torch.manual_seed(5)
    fused = getattr(modules, cls)(cin, cout, 3, padding=1, **kw).cuda().to(dtype)
    torch.nn.init.normal_(fused.deform_params.weight, std=0.08)          # non-trivial deformation
    if fused.deform_params.bias is not None:
        torch.nn.init.normal_(fused.deform_params.bias, std=0.2)
    plain = copy.deepcopy(fused)
    plain.fused_head = False
    assert fused.fused_head
    return fused, plain


def run(layer, x, gy):
    x = x.detach().clone().requires_grad_()
    y = layer(x)
    y.backward(gy)
    torch.cuda.synchronize()
    return [y.detach(), x.grad] + [p.grad for p in layer.parameters()]


CASES = [
    # class, Cin, Cout, constructor kwargs
    ("MDConv3d", 64, 64, dict(offset_groups=1)),
    ("MDConv3d", 128, 64, dict(offset_groups=2, activation="tanh")),
    ("MDConv3d", 64, 64, dict(activation="relu")),
    ("MDConv3d", 64, 64, dict(activation="none")),
    ("DConv3d", 64, 64, dict()),
    ("XYZSizeConditionedMDConv3d", 256, 64, dict(offset_groups=8)),                      # 32 channels per group
    ("XYZSizeConditionedMDConv3d", 64, 64, dict(size_activation="relu")),
    ("XYSizeConditionedDConv3d", 64, 64, dict(size_activation="relu_plus_one")),
    ("SizeConditionedMDConv3d", 64, 64, dict(size_activation="linear")),
    ("XXZSizeConditionedMDConv3d", 64, 128, dict(size_activation="elu")),
]


@pytest.mark.parametrize("ci", range(len(CASES)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_fused_head_matches_unfused_layer(mods, ci, dtype):
    from d2conv3d_b200 import _lib
    cls, cin, cout, kw = CASES[ci]
    if dtype == torch.float64:
        cin, cout = cin // 8, cout // 8            # the CUDA-core tier; keep it small
        if kw.get("offset_groups", 1) > cin:
            kw = dict(kw, offset_groups=cin)
    fused, plain = make_pair(mods, cls, cin, cout, dtype, **kw)
    g = torch.Generator().manual_seed(9)
    x = torch.randn((2, cin, 3, 9, 10), generator=g, dtype=dtype).cuda()
    if fused.field_mode is not None and fused.size_activation == "linear":
        with torch.no_grad():                       # a raw field must be a sensible scale by itself
            fused.deform_params.bias[:fused.offset_channels] += 1.5
            plain.deform_params.bias[:plain.offset_channels] += 1.5
    gy = torch.randn((2, cout, 3, 9, 10), generator=g, dtype=dtype).cuda()
    _lib.profile_read(); _lib.profile_enable(True)
    got = run(fused, x, gy)
    _lib.profile_enable(False)
    phases = {n for n, _ in _lib.profile_read()}
    if dtype == torch.float32:
        assert "fwd_sm100_fused" in phases and "bwd_sample_grad" in phases, phases     # the truly fused route
    want = run(plain, x, gy)
    tol = 1e-4 if dtype == torch.float32 else 1e-10
    names = ["y", "grad_x"] + [n for n, _ in fused.named_parameters()]
    for name, a, b in zip(names, got, want):
        err = float((a - b).abs().max()) / max(float(b.abs().max()), 1e-30)
        assert err <= tol, (cls, name, err)


def _kernel_names(fn):
    from torch.profiler import ProfilerActivity, profile
    fn()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        fn()
        torch.cuda.synchronize()
    return [e.name for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]


ELEMENTWISE = ("sigmoid", "elu_kernel", "tanh", "elementwise", "copy", "CatArray", "clamp")


@pytest.mark.parametrize("cls", ["MDConv3d", "XYZSizeConditionedMDConv3d"])
def test_no_elementwise_kernel_between_predictor_and_layer(mods, cls):
    """Kernel list of one forward: the unfused layer runs activation / copy kernels of PyTorch between the
    predictor convolution and the op, the fused one none.  (The predictor has no bias here, so that cuDNN's own
    bias epilogue cannot be mistaken for one.)"""
    fused, plain = make_pair(mods, cls, 64, 64, torch.float32, bias=False)
    x = torch.randn(1, 64, 3, 9, 10, device="cuda")
    with torch.no_grad():
        names_plain = _kernel_names(lambda: plain(x))
        names_fused = _kernel_names(lambda: fused(x))
    if not names_plain or not names_fused:
        pytest.skip("the profiler reported no device kernels on this machine")
    hits = lambda names: [n for n in names if any(k in n for k in ELEMENTWISE)]
    assert hits(names_plain), f"detector saw no elementwise kernel in the unfused layer: {names_plain}"
    assert not hits(names_fused), hits(names_fused)
    assert any("sample_records" in n for n in names_fused) and any("fwd_sm100" in n for n in names_fused), names_fused
