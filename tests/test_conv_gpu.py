"""tcgen05 stem convolution (7 x 7 / 2, 3 -> 64) and fused partition execution against plain PyTorch in fp32."""
import copy

import pytest
import torch
import torch.nn.functional as F
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,h,w", [(2, 64, 64), (3, 224, 224), (5, 96, 40), (1, 8, 8), (150, 16, 16)])
def test_stem_conv_matches_fp32_reference(n, h, w):
    from tspipe_b200.ops import conv, gemm
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    x = torch.randn(n, 3, h, w, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    weight = (torch.randn(64, 3, 7, 7, device=dev) * 0.1).requires_grad_()
    assert conv.eligible(x)
    y, sums = conv.stem_conv(x, weight)
    gemm.check_status()
    wr = weight.detach().bfloat16().float().requires_grad_()
    ref = F.conv2d(x.float(), wr, stride=2, padding=3)
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    yf = y.float()
    torch.testing.assert_close(sums[:64], yf.sum((0, 2, 3)), rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(sums[64:], (yf * yf).sum((0, 2, 3)), rtol=1e-3, atol=1e-2)
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float())
    torch.testing.assert_close(weight.grad, wr.grad, rtol=5e-2, atol=5e-2 * wr.grad.abs().max().item())


def test_fused_partition_matches_plain_sequential():
    """conv1 -> bn1 -> relu -> maxpool -> linear head -> bn1d -> relu run through FusedSequential give the same
    outputs, gradients and BatchNorm statistics as the plain modules."""
    from tspipe_b200.batchnorm import DeferredBatchNorm
    from tspipe_b200.ops import gemm
    from tspipe_b200.ops.pool import MaxPool3x3s2
    from tspipe_b200.runtime.fuse import FusedSequential, fuse_partition
    torch.manual_seed(1)
    dev = torch.device("cuda", 0)

    def build():
        return nn.Sequential(nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False), DeferredBatchNorm(64, chunks=10 ** 9),
                             nn.ReLU(), MaxPool3x3s2(), nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(64, 32),
                             DeferredBatchNorm(32, chunks=10 ** 9), nn.ReLU()).to(dev).to(memory_format=torch.channels_last)
    plain = build()
    fused = copy.deepcopy(plain)
    fuse_partition(fused)
    assert isinstance(fused, FusedSequential) and list(fused.state_dict()) == list(plain.state_dict())
    x = torch.randn(16, 3, 64, 64, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    outs = []
    for net in (plain, fused):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = net(x)
        y.float().square().mean().backward()
        outs.append(y)
    gemm.check_status()
    torch.testing.assert_close(outs[1].float(), outs[0].float(), rtol=3e-2, atol=3e-2)
    for (k, p), q in zip(plain.named_parameters(), fused.parameters()):
        torch.testing.assert_close(q.grad, p.grad, rtol=5e-2, atol=5e-2 * max(p.grad.abs().max().item(), 1e-3), msg=k)
    torch.testing.assert_close(fused[1].sum, plain[1].sum, rtol=1e-2, atol=1.0)
    torch.testing.assert_close(fused[1].sum_squares, plain[1].sum_squares, rtol=1e-2, atol=1.0)


def test_stem_conv_statistics_per_group_of_images():
    from tspipe_b200.ops import conv, gemm
    torch.manual_seed(2)
    dev = torch.device("cuda", 0)
    x = torch.randn(6, 3, 32, 32, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    x[3:] *= 3.0
    weight = torch.randn(64, 3, 7, 7, device=dev) * 0.1
    y, sums = conv.stem_conv(x, weight, segments=2)
    gemm.check_status()
    yf = y.float()
    sums = sums.view(2, 128)
    for g, part in enumerate((yf[:3], yf[3:])):
        torch.testing.assert_close(sums[g, :64], part.sum((0, 2, 3)), rtol=1e-3, atol=1e-2)
        torch.testing.assert_close(sums[g, 64:], (part * part).sum((0, 2, 3)), rtol=1e-3, atol=1e-2)
