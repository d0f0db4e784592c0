"""ir-CSN bottleneck block: same function (forward and gradients) as the block built with
nn.Conv3d(groups=channels) in place of the depthwise op, as the reference falls back to when the extension is
missing (network/backbone/resnet.py:11-16)."""
import pytest
import torch
import torch.nn as nn

from d2conv3d_b200.backbone import IrBottleneck3d


def test_structure_cpu():
    b = IrBottleneck3d(64, 16, stride=(1, 2, 2))
    assert b.conv2.groups == 16 and b.conv2.bias is None and b.conv3.out_channels == 64
    assert [n for n, _ in b.named_children()][:6] == ["conv1", "bn1", "conv2", "bn2", "conv3", "bn3"]


@pytest.mark.gpu
@pytest.mark.parametrize("stride,dilation,ckpt", [(1, 1, False), ((1, 2, 2), 1, False), (1, 2, True)])
def test_block_matches_grouped_conv_block(stride, dilation, ckpt):
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.manual_seed(4)
    ds = None
    if stride != 1:
        ds = nn.Sequential(nn.Conv3d(64, 64, 1, stride=stride, bias=False), nn.BatchNorm3d(64))
    ours = IrBottleneck3d(64, 16, stride=stride, dilation=dilation, downsample=ds, use_checkpoint=ckpt).cuda()
    import copy
    ref = IrBottleneck3d(64, 16, stride=stride, dilation=dilation, downsample=copy.deepcopy(ds),
                         depthwise=nn.Conv3d).cuda()
    ref.load_state_dict(ours.state_dict())
    x1 = torch.randn(2, 64, 4, 10, 12, device="cuda").requires_grad_()
    x2 = x1.detach().clone().requires_grad_()
    y1, y2 = ours(x1), ref(x2)
    assert float((y1 - y2).abs().max()) <= 1e-5 * float(y2.abs().max())
    g = torch.randn_like(y1)
    y1.backward(g); y2.backward(g)
    assert float((x1.grad - x2.grad).abs().max()) <= 1e-4 * float(x2.grad.abs().max())
    for (n, p1), (_, p2) in zip(ours.named_parameters(), ref.named_parameters()):
        # batch-norm parameter gradients are sums of thousands of O(1) terms that cancel to ~1e-2: allow the
        # fp32 summation noise of those terms on top of the relative bound
        assert float((p1.grad - p2.grad).abs().max()) <= 1e-4 * float(p2.grad.abs().max()) + 5e-5, n
