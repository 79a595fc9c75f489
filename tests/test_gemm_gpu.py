"""tcgen05 / TMEM / TMA GEMM against an fp32 PyTorch product of the same bf16-rounded operands."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("two_cta", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 256, 128), (384, 512, 320), (200, 136, 72), (300, 100, 64),
                                   (1024, 768, 768), (4096, 4096, 256)])
def test_matmul_nt_matches_fp32_reference(m, n, k, two_cta):
    """Both kernels (one CTA per tile; CTA pair per tile with TMA-store epilogue), ragged edges included:
    (300, 100) has a bf16 row pitch that is no multiple of 16 bytes, which takes the direct-store epilogue."""
    from tspipe_b200.ops import gemm
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    a = torch.randn(m, k, device=dev).bfloat16()
    b = torch.randn(n, k, device=dev).bfloat16()
    c = gemm.matmul_nt(a, b, out_dtype=torch.float32, two_cta=two_cta)
    gemm.check_status()
    ref = a.float() @ b.float().t()
    torch.testing.assert_close(c, ref, rtol=1e-3, atol=1e-2 * (k ** 0.5) / 8)
    c16 = gemm.matmul_nt(a, b, two_cta=two_cta)
    gemm.check_status()
    torch.testing.assert_close(c16.float(), ref, rtol=2e-2, atol=0.1 * (k ** 0.5) / 8)


@pytest.mark.parametrize("two_cta", [False, True])
def test_bias_gelu_epilogue(two_cta):
    from tspipe_b200.ops import gemm
    torch.manual_seed(1)
    dev = torch.device("cuda", 0)
    a = (torch.randn(512, 256, device=dev) * 0.5).bfloat16()
    b = (torch.randn(384, 256, device=dev) * 0.1).bfloat16()
    bias = torch.randn(384, device=dev)
    y = gemm.matmul_nt(a, b, bias, gelu=True, out_dtype=torch.float32, two_cta=two_cta)
    gemm.check_status()
    ref = F.gelu(a.float() @ b.float().t() + bias)
    torch.testing.assert_close(y, ref, rtol=1e-3, atol=1e-3)


def test_linear_autograd_and_info_nce():
    from tspipe_b200.ops import fused, gemm
    torch.manual_seed(2)
    dev = torch.device("cuda", 0)
    x = torch.randn(4, 64, 128, device=dev, requires_grad=True)
    w = (torch.randn(256, 128, device=dev) * 0.1).requires_grad_()
    bias = torch.randn(256, device=dev, requires_grad=True)
    y = gemm.linear(x, w, bias)
    y.float().pow(2).mean().backward()
    gemm.check_status()
    xr, wr, br = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_(), bias.detach().clone().requires_grad_()
    yr = F.linear(xr, wr, br)
    yr.pow(2).mean().backward()
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(x.grad, xr.grad, rtol=5e-2, atol=2e-4)
    torch.testing.assert_close(w.grad, wr.grad, rtol=5e-2, atol=2e-4)
    q = torch.randn(512, 256, device=dev, requires_grad=True)
    k = torch.randn(512, 256, device=dev)
    loss = fused.info_nce_loss(q, k, 0.2)
    loss.backward()
    gemm.check_status()
    qr = q.detach().clone().requires_grad_()
    logits = F.normalize(qr, dim=1) @ F.normalize(k, dim=1).t() / 0.2
    ref = F.cross_entropy(logits, torch.arange(512, device=dev)) * 0.4
    ref.backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q.grad, qr.grad, rtol=1e-1, atol=2e-4)


@pytest.mark.parametrize("rows,k,n", [((4, 64), 128, 256), ((3, 197), 768, 2304), ((1000,), 64, 64), ((5, 130), 3072, 768)])
def test_linear_forward_and_both_backward_products_on_tcgen05(rows, k, n):
    """``ops.linear.linear`` under bf16 autocast (the default path of the transformer blocks and heads): output, dX,
    dW (added in place into an existing fp32 gradient) and db against fp32 F.linear on the same bf16-rounded
    operands; ragged row counts included."""
    from tspipe_b200.ops import gemm
    from tspipe_b200.ops.linear import linear
    torch.manual_seed(5)
    dev = torch.device("cuda", 0)
    x = torch.randn(*rows, k, device=dev, requires_grad=True)
    w = (torch.randn(n, k, device=dev) * 0.05).requires_grad_()
    bias = torch.randn(n, device=dev, requires_grad=True)
    w.grad = torch.full_like(w, 0.5)                 # an existing gradient: the kernel accumulates into it
    before = gemm._f.LAUNCHES
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert gemm.eligible(x, w)
        y = linear(x, w, bias)
    g = torch.randn_like(y)
    y.backward(g)
    gemm.check_status()
    assert gemm._f.LAUNCHES - before >= 3            # forward GEMM, dX, dW (+ bias gradient) are own launches
    xr = x.detach().bfloat16().float().requires_grad_()
    wr = w.detach().bfloat16().float().requires_grad_()
    br = bias.detach().clone().requires_grad_()
    yr = F.linear(xr, wr, br)
    yr.backward(g.float())
    scale = (k ** 0.5) / 8
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=0.05 * scale)
    torch.testing.assert_close(x.grad, xr.grad, rtol=3e-2, atol=3e-2 * max(xr.grad.abs().max().item(), 1e-3))
    torch.testing.assert_close(w.grad - 0.5, wr.grad, rtol=3e-2, atol=3e-2 * wr.grad.abs().max().item())
    torch.testing.assert_close(bias.grad, br.grad, rtol=2e-2, atol=2e-2 * br.grad.abs().max().item())
