"""tcgen05 convolutions (stem 7 x 7 / 2, implicit-GEMM 1x1 / 3x3) and fused partition execution against plain PyTorch
in fp32."""
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


# (input shape NCHW, cout, kernel, stride, segments)
IGEMM_CASES = [
    ((4, 64, 16, 16), 256, 1, 1, 1),      # 1x1: plain GEMM over 1024 pixels
    ((8, 256, 8, 8), 64, 1, 1, 2),        # narrow output, two view segments
    ((3, 128, 10, 10), 64, 1, 1, 1),      # 300 pixels: ragged last tile (no statistics possible)
    ((4, 64, 14, 14), 64, 3, 1, 2),       # 3x3: boxes of 14 x 7 pixels, odd number of (tap, ci) blocks
    ((2, 64, 9, 9), 128, 3, 1, 1),        # odd width: 81-pixel boxes (zero rows in the weight-gradient K loop)
    ((8, 128, 7, 7), 128, 3, 1, 2),       # 7 x 7 images: two images per box
    ((2, 64, 12, 12), 128, 3, 2, 1),      # stride 2 through the parity views
    ((2, 128, 56, 56), 128, 3, 2, 2),     # ResNet-50 layer2 shape: 28 x 4 boxes
    ((2, 128, 8, 8), 256, 1, 2, 1),       # 1x1 stride 2 (downsample branch)
    ((2, 256, 56, 56), 64, 1, 1, 2),      # ResNet-50 layer1 conv1
    ((2, 512, 16, 8), 1024, 1, 1, 2),
    ((1, 64, 130, 6), 64, 3, 1, 1),       # wider than one box
]


@pytest.mark.parametrize("shape,cout,k,stride,segs", IGEMM_CASES)
def test_igemm_convolution_forward_backward_and_statistics(shape, cout, k, stride, segs):
    """Implicit-GEMM convolution on tcgen05: output, per-segment channel statistics, data and weight gradient against
    F.conv2d in fp32 (same bf16-rounded operands)."""
    from tspipe_b200.ops import conv, gemm
    torch.manual_seed(3)
    dev = torch.device("cuda", 0)
    x = torch.randn(shape, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last).requires_grad_()
    m = nn.Conv2d(shape[1], cout, k, stride=stride, padding=(k - 1) // 2, bias=False).to(dev)
    m = m.to(memory_format=torch.channels_last)
    assert conv.igemm_eligible(m, x)
    conv.clear_weight_cache()
    y, sums = conv.conv2d(x, m.weight, stride, want_sums=True, segments=segs)
    gemm.check_status()
    xr = x.detach().float().requires_grad_()
    wr = m.weight.detach().bfloat16().float().requires_grad_()
    ref = F.conv2d(xr, wr, stride=stride, padding=(k - 1) // 2)
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    yf = y.float()
    if sums is not None:
        sums = sums.view(segs, 2, cout)
        for g, part in enumerate(yf.chunk(segs)):
            torch.testing.assert_close(sums[g, 0], part.sum((0, 2, 3)), rtol=1e-3, atol=2e-2)
            torch.testing.assert_close(sums[g, 1], (part * part).sum((0, 2, 3)), rtol=1e-3, atol=2e-2)
    else:
        pixels = shape[0] // segs * ref.shape[2] * ref.shape[3]
        assert k == 1 and stride == 1 and pixels % 128 != 0     # the only case without statistics: ragged 1x1 tiles
    g = torch.randn_like(y)
    y.backward(g)
    gemm.check_status()
    ref.backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2 * max(xr.grad.abs().max().item(), 1.0))
    torch.testing.assert_close(m.weight.grad, wr.grad, rtol=5e-2, atol=5e-2 * wr.grad.abs().max().item())
    # a second backward ADDS into the existing fp32 gradient (the kernel accumulates in place)
    y2, _ = conv.conv2d(x, m.weight, stride)
    y2.backward(g)
    gemm.check_status()
    torch.testing.assert_close(m.weight.grad, 2 * wr.grad, rtol=5e-2, atol=1e-1 * wr.grad.abs().max().item())


def test_bottleneck_on_igemm_convolutions_matches_library_path():
    from tspipe_b200.batchnorm import DeferredBatchNorm
    from tspipe_b200.models.resnet import Bottleneck
    from tspipe_b200.ops import conv, gemm
    torch.manual_seed(4)
    dev = torch.device("cuda", 0)
    down = nn.Sequential(nn.Conv2d(256, 512, 1, stride=2, bias=False), nn.BatchNorm2d(512))
    blk = DeferredBatchNorm.convert_deferred_batch_norm(Bottleneck(256, 128, 2, down), chunks=10 ** 9).to(dev)
    blk = blk.to(memory_format=torch.channels_last)
    x = torch.randn(8, 256, 16, 16, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    outs, grads = [], []
    for flag in (False, True):
        conv.set_igemm(flag)
        conv.clear_weight_cache()
        try:
            xi = x.clone().requires_grad_()
            blk.zero_grad()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = blk(xi)
            y.float().square().mean().backward()
        finally:
            conv.set_igemm(True)
        outs.append(y.float())
        grads.append([xi.grad.float()] + [p.grad.clone() for p in blk.parameters()])
    gemm.check_status()
    torch.testing.assert_close(outs[1], outs[0], rtol=3e-2, atol=3e-2)
    for a, b in zip(grads[1], grads[0]):
        torch.testing.assert_close(a, b, rtol=5e-2, atol=5e-2 * max(b.abs().max().item(), 1e-3))
