"""Fused attention forward on tcgen05 (and the contrastive loss built on it) against plain PyTorch in fp32."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _ref(q, k, v, scale):
    s = (q.float() @ k.float().transpose(-1, -2)) * scale
    return torch.softmax(s, -1) @ v.float(), torch.logsumexp(s, -1)


@pytest.mark.parametrize("b,h,nq,nk", [(2, 3, 197, 197), (1, 2, 64, 64), (1, 1, 128, 128), (2, 2, 300, 520), (3, 12, 50, 197)])
def test_flash_forward_head_dim_64(b, h, nq, nk):
    """Interleaved qkv layout as the ViT blocks produce it ([B, N, 3, H, 64] viewed as [B, H, N, 64])."""
    from tspipe_b200.ops import attention, gemm
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    n = max(nq, nk)
    qkv = (torch.randn(b, n, 3, h, 64, device=dev) * 1.5).bfloat16()
    q, k, v = qkv.permute(2, 0, 3, 1, 4)
    q, k, v = q[:, :, :nq], k[:, :, :nk], v[:, :, :nk]
    assert attention.flash_eligible(q, k, v)
    o, lse = attention.flash_fwd(q, k, v, want_lse=True)
    gemm.check_status()
    ro, rl = _ref(q, k, v, 1 / math.sqrt(64))
    assert o.shape == (b, h, nq, 64)
    assert o.transpose(1, 2).reshape(b, nq, h * 64).is_contiguous()
    torch.testing.assert_close(o.float(), ro, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, rl, rtol=1e-3, atol=1e-2)


def test_attention_dispatch_and_vit_block_without_grad():
    """A ViT block gives the same result through the three attention paths: tcgen05 kernel (no gradient needed,
    opt-in), the library's fused attention on unbound q / k / v, and the packed-qkv library entry point."""
    from tspipe_b200.models.vit import CONFIGS, Block
    from tspipe_b200.ops import attention, gemm
    torch.manual_seed(1)
    dev = torch.device("cuda", 0)
    blk = Block(CONFIGS["vit_base"]).to(dev)
    x = torch.randn(4, 197, 768, device=dev)
    try:
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            attention.set_qkv_mode("packed")
            attention.set_packed(False)
            attention.set_tcgen05(True)
            y = blk(x)                                   # tcgen05 attention
            attention.set_tcgen05(False)
            y_ref = blk(x)                               # library attention on unbound q, k, v
            attention.set_packed(None)
            y_packed = blk(x)                            # packed entry point when the library supports this GPU
            attention.set_qkv_mode("split")
            y_split = blk(x)                             # three projection GEMMs + library attention
    finally:
        attention.set_tcgen05(False)
        attention.set_packed(None)
        attention.set_qkv_mode("split")
    gemm.check_status()
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(y_packed.float(), y_ref.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(y_split.float(), y_ref.float(), rtol=3e-2, atol=3e-2)
    grads = {}
    for mode in ("split", "packed"):                      # with gradients, both ways of forming q, k, v
        attention.set_qkv_mode(mode)
        try:
            xg = x.clone().requires_grad_()
            blk.zero_grad()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                blk(xg).float().sum().backward()
            grads[mode] = (xg.grad.clone(), blk.attn.qkv.weight.grad.clone())
        finally:
            attention.set_qkv_mode("split")
    for a, b in zip(grads["split"], grads["packed"]):
        torch.testing.assert_close(a, b, rtol=5e-2, atol=5e-2 * b.abs().max().item())


def test_patch_embedding_as_gemm_matches_convolution():
    from tspipe_b200.models.vit import CONFIGS, PatchEmbed
    torch.manual_seed(5)
    dev = torch.device("cuda", 0)
    pe = PatchEmbed(CONFIGS["vit_base"]).to(dev)
    for fmt in (torch.contiguous_format, torch.channels_last):
        x = torch.randn(3, 3, 224, 224, device=dev).contiguous(memory_format=fmt).requires_grad_()
        y = pe(x)
        ref = pe.proj(x).flatten(2).transpose(1, 2)
        torch.testing.assert_close(y, ref, rtol=2e-3, atol=2e-3)     # TF32 may be on for either path
        g = torch.randn_like(y)
        gw = torch.autograd.grad(y, pe.proj.weight, g, retain_graph=True)[0]
        gw_ref = torch.autograd.grad(ref, pe.proj.weight, g)[0]
        torch.testing.assert_close(gw, gw_ref, rtol=2e-3, atol=2e-3 * gw_ref.abs().max().item())


@pytest.mark.parametrize("n", [128, 1024, 4096])
def test_fused_contrastive_loss_matches_cross_entropy(n):
    """Loss value and gradient from one fused pass (V = K, scores bounded by 1/T) vs normalize + matmul + CE."""
    from tspipe_b200.ops import fused, gemm
    torch.manual_seed(2)
    dev = torch.device("cuda", 0)
    temp = 0.2
    q = torch.randn(n, 256, device=dev, requires_grad=True)
    k = torch.randn(n, 256, device=dev)
    k[: n // 2] += 0.5 * q.detach()[: n // 2]        # some positives that actually align
    loss = fused.info_nce_loss(q, k, temp)
    loss.backward()
    gemm.check_status()
    qr = q.detach().clone().requires_grad_()
    logits = F.normalize(qr, dim=1) @ F.normalize(k, dim=1).t() / temp
    ref = F.cross_entropy(logits, torch.arange(n, device=dev)) * (2 * temp)
    ref.backward()
    torch.testing.assert_close(loss, ref, rtol=5e-3, atol=5e-3)
    torch.testing.assert_close(q.grad, qr.grad, rtol=5e-2, atol=5e-2 * qr.grad.abs().max().item())
    gemm.set_fused_nce(False)
    try:
        q2 = q.detach().clone().requires_grad_()
        unfused = fused.info_nce_loss(q2, k, temp)
    finally:
        gemm.set_fused_nce(True)
    torch.testing.assert_close(loss, unfused, rtol=5e-3, atol=5e-3)
