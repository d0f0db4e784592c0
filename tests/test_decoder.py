"""Decoder composition (d2conv3d_b200/decoder.py).  CPU: structure, parameter shapes, pyramid shapes.
GPU: at initialisation the dilation-field + mask layers reduce to 0.5 * conv3d (zero-initialised predictor:
field = elu(0)+1 = 1 -> zero offsets, mask = sigmoid(0) = 0.5; the identity the reference's module tests use,
ops/dconv-native/test/test_modules.py:48-67), so the whole deformable decoder must equal a plain-conv decoder with
those weights halved; and clips are independent (sharding by clip changes nothing)."""
import pytest
import torch

from d2conv3d_b200 import decoder as dec
from d2conv3d_b200.dconv_native import modules


def small(conv):
    torch.manual_seed(3)
    return dec.Decoder(widths=(64, 64, 128, 128), channels=64, num_classes=2, conv=conv, offset_groups=2)


def test_structure_and_shapes_cpu():
    d = small("XYZSizeConditionedDCNv2")
    assert d.converted == 15                                   # 3 refine blocks x 5 convolutions
    layer = d.rf1.convFS1[0]
    assert isinstance(layer, modules.XYZSizeConditionedMDConv3d)
    assert layer.deform_params.out_channels == 3 + 2 * 27      # 3 field channels + one mask per (group, tap)
    assert isinstance(d.gc.conv_l1, torch.nn.Conv3d) and d.gc.conv_l1.kernel_size == (1, 7, 1)
    assert dec.pyramid_shapes(32) == [(32, 256, 8, 120, 214), (32, 512, 8, 60, 107), (32, 1024, 8, 30, 54),
                                      (32, 2048, 8, 15, 27)]
    assert small(None).converted == 0


def feats(B, dev):
    g = torch.Generator().manual_seed(5)
    shapes = [(B, 64, 2, 12, 16), (B, 64, 2, 6, 8), (B, 128, 2, 3, 4), (B, 128, 2, 2, 2)]
    return [torch.relu(torch.randn(s, generator=g)).to(dev) for s in shapes]


@pytest.mark.gpu
def test_deformable_decoder_at_init_equals_halved_plain_decoder():
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    d = small("XYZSizeConditionedDCNv2").cuda().eval()
    p = small(None).cuda().eval()
    sd = {}
    for k, v in d.state_dict().items():
        if ".deform_params." in k:
            continue
        if ".deform_conv." in k:
            k2 = k.replace(".deform_conv.", ".")
            sd[k2] = v * 0.5 if k.endswith("weight") else v
        else:
            sd[k] = v
    p.load_state_dict(sd)
    with torch.no_grad():
        a = d(*feats(2, "cuda"))
        b = p(*feats(2, "cuda"))
    assert a.shape == (2, 2, 2, 48, 64)
    assert float((a - b).abs().max() / b.abs().max()) <= 1e-4


@pytest.mark.gpu
def test_clips_are_independent():
    torch.backends.cudnn.allow_tf32 = False          # cuDNN may pick different TF32 algorithms per batch size
    torch.backends.cuda.matmul.allow_tf32 = False
    d = small("XYZSizeConditionedDCNv2").cuda().eval()
    for m in d.modules():                      # non-trivial deformation: random predictor weights
        if isinstance(m, modules.XYZSizeConditionedMDConv3d):
            # small predictor weights: with large random ones the predicted field makes every layer's output
            # very sensitive to its input, and the last-bit differences between two runs (partial tiles are
            # combined with atomics, in any order) are amplified layer by layer
            torch.nn.init.normal_(m.deform_params.weight, std=0.005)
    f = feats(3, "cuda")
    with torch.no_grad():
        whole = d(*f)
        parts = torch.cat([d(*[t[i:i + 1] for t in f]) for i in range(3)])
    err = float((whole - parts).abs().max() / whole.abs().max())
    assert err <= 1e-4, err


@pytest.mark.gpu
@pytest.mark.parametrize("shape,groups", [((1, 64, 2, 12, 16), 1), ((3, 48, 3, 5, 7), 4), ((2, 8, 1, 3, 5), 2)])
def test_fused_relu_group_norm_matches_torch(shape, groups):
    from d2conv3d_b200 import _lib
    g = torch.Generator().manual_seed(9)
    x = torch.randn(shape, generator=g).cuda() * 3 + 0.5
    w = torch.randn(shape[1], generator=g).cuda()
    b = torch.randn(shape[1], generator=g).cuda()
    y = _lib.act_group_norm(x, w, b, groups, 1e-5, relu=True)
    ref = torch.nn.functional.group_norm(torch.relu(x), groups, w, b, 1e-5)
    assert float((y - ref).abs().max()) <= 1e-5 * max(1.0, float(ref.abs().max()))
    y2 = _lib.act_group_norm(x, None, None, groups, 1e-5, relu=False)
    ref2 = torch.nn.functional.group_norm(x, groups, None, None, 1e-5)
    assert float((y2 - ref2).abs().max()) <= 1e-5 * max(1.0, float(ref2.abs().max()))


def test_clip_shares_cover_the_job():
    import bench
    for total in (32, 7, 1):
        for world in (1, 2, 4, 8):
            shares = [bench.decoder_share(total, r, world) for r in range(world)]
            assert sum(shares) == total and max(shares) - min(shares) <= 1


@pytest.mark.gpu
@pytest.mark.parametrize("shape,groups,relu", [((2, 64, 2, 12, 16), 1, True), ((3, 48, 3, 5, 7), 4, True),
                                                ((2, 8, 1, 3, 5), 2, False)])
def test_fused_relu_group_norm_backward_matches_torch(shape, groups, relu):
    from d2conv3d_b200 import _lib
    g = torch.Generator().manual_seed(10)
    x = (torch.randn(shape, generator=g) * 2 + 0.3).cuda().requires_grad_()
    w = torch.randn(shape[1], generator=g).cuda().requires_grad_()
    b = torch.randn(shape[1], generator=g).cuda().requires_grad_()
    gy = torch.randn(shape, generator=g).cuda()
    y = _lib.act_group_norm(x, w, b, groups, 1e-5, relu=relu)
    y.backward(gy)
    got = [x.grad.clone(), w.grad.clone(), b.grad.clone()]
    x.grad = w.grad = b.grad = None
    ref = torch.nn.functional.group_norm(torch.relu(x) if relu else x, groups, w, b, 1e-5)
    ref.backward(gy)
    for a, r, n in zip(got, (x.grad, w.grad, b.grad), ("grad_x", "grad_weight", "grad_bias")):
        assert float((a - r).abs().max()) <= 1e-4 * max(1.0, float(r.abs().max())), n


@pytest.mark.gpu
def test_decoder_trains_one_step():
    """Forward + backward through the whole decoder (deformable layers, fused norm) gives finite gradients for
    every parameter, and matches the plain-conv decoder at initialisation (where both are the same function)."""
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    d = small("XYZSizeConditionedDCNv2").cuda().train()
    out = d(*feats(1, "cuda"))
    out.square().mean().backward()
    for n, p_ in d.named_parameters():
        assert p_.grad is not None and torch.isfinite(p_.grad).all(), n
