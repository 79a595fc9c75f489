"""Scaled dot-product attention ``softmax(Q K^T / sqrt(d) + mask) V`` for [B, H, N, D] tensors.

The reference models run it unfused - two batched GEMMs, a softmax and a dropout
(timm ``Attention`` in `benchmarks/moco-v3/vits.py`, HF ``BertSelfAttention`` in
`benchmarks/distilbert/bert.py`).  Here it is one fused call; ``mask`` is an additive or boolean
key-padding mask broadcastable to [B, 1, 1, N] / [B, H, N, N].

Forward passes that need no gradient (the teacher / momentum encoder) with head dimension 64 and no mask run on
the tcgen05 kernel of ``csrc/attn_tcgen05.cu`` (:func:`flash_fwd`); everything else goes to the library's fused
attention, which also provides the backward.
"""
from __future__ import annotations

import ctypes as _c
import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

# The tcgen05 kernel launches one CTA per (128-query tile, head): at ViT sizes (197 tokens) that is two key tiles per
# CTA and the per-CTA start-up dominates (343 us against the library's 105 us on [256, 12, 197, 64]), so it is opt-in
# for attention; the contrastive loss (long key loops) uses it by default.
_TCGEN05 = False


def set_tcgen05(flag: bool) -> None:
    global _TCGEN05
    _TCGEN05 = bool(flag)


_PACKED = {"state": None}     # None = not probed yet, True / False = usable or not

# How the ViT blocks form q, k, v: "packed" = one projection GEMM and the packed-qkv library attention; "split" =
# three projection GEMMs on slices of the weight and the generic fused attention (no packed tensor, hence no
# concatenation of dq, dk, dv in the backward either).
_QKV_MODE = "split"      # measured on MoCo-v3 ViT-B, 256 samples per GPU: 114.8 ms per step against 121.3 ms for "packed"


def set_qkv_mode(mode: str) -> None:
    global _QKV_MODE
    assert mode in ("packed", "split")
    _QKV_MODE = mode


def qkv_mode() -> str:
    return _QKV_MODE


def project_qkv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], heads: int):
    """``q, k, v`` as ``[B, H, N, D]`` views from the fused projection parameters ``weight [3C, C]``, ``bias [3C]``.
    On CUDA in "split" mode this is three GEMMs on slices of the parameters, so that no packed qkv tensor exists
    whose gradient autograd would have to assemble from dq, dk and dv; otherwise one GEMM and an unbind."""
    from .linear import linear
    b, n, c = x.shape
    if x.is_cuda and _QKV_MODE == "split":
        return tuple(linear(x, weight[i * c:(i + 1) * c], None if bias is None else bias[i * c:(i + 1) * c])
                     .view(b, n, heads, c // heads).transpose(1, 2) for i in range(3))
    qkv = linear(x, weight, bias).reshape(b, n, 3, heads, c // heads)
    return tuple(qkv.permute(2, 0, 3, 1, 4))


def set_packed(flag: Optional[bool]) -> None:
    """Force (True / False) or re-probe (None) the packed-qkv library attention."""
    _PACKED["state"] = flag


def packed_attention(qkv: torch.Tensor) -> Optional[torch.Tensor]:
    """Attention on the packed projection output ``qkv [B, N, 3, H, D]`` -> ``[B, N, H, D]`` through the
    flash-attn library's packed entry point, or None when that is not usable here.  Compared with unbinding q, k, v
    for the generic fused attention this avoids two full-size copies per block and step: the concatenation of
    dq, dk, dv that autograd builds for the packed tensor, and the ``[B, H, N, D] -> [B, N, H * D]`` repacking of
    the output."""
    if _PACKED["state"] is False or not (qkv.is_cuda and qkv.dtype in (torch.bfloat16, torch.float16)):
        return None
    if qkv.shape[-1] > 256 or qkv.shape[-1] % 8:
        return None
    try:
        from flash_attn import flash_attn_qkvpacked_func
        if _PACKED["state"] is None:
            probe = torch.randn(1, 16, 3, 1, 64, device=qkv.device, dtype=torch.bfloat16)
            ref = F.scaled_dot_product_attention(*(t.transpose(1, 2) for t in probe.unbind(2))).transpose(1, 2)
            ok = torch.allclose(flash_attn_qkvpacked_func(probe).float(), ref.float(), rtol=3e-2, atol=3e-2)
            _PACKED["state"] = bool(ok)
            if not ok:
                return None
        return flash_attn_qkvpacked_func(qkv)
    except Exception:   # noqa: BLE001 - library missing or not built for this GPU: use the generic path
        _PACKED["state"] = False
        return None


def _strides3(t: torch.Tensor):
    """(row, head, batch) element strides of a [B, H, N, D] tensor as a ctypes array."""
    return (_c.c_int64 * 3)(t.stride(2), t.stride(1), t.stride(0))


def flash_eligible(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    if not (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16 and q.dim() == k.dim() == v.dim() == 4):
        return False
    d, dv = q.shape[-1], v.shape[-1]
    if (d, dv) not in ((64, 64), (256, 256)):
        return False
    if d == 256 and not (k.data_ptr() == v.data_ptr() and k.stride() == v.stride()):
        return False
    if q.shape[0] * q.shape[1] > 65535 or k.shape[2] < 1:
        return False
    for t in (q, k, v):
        if t.stride(-1) != 1 or t.data_ptr() % 16 or any(s % 8 for s in t.stride()[:-1]):
            return False
    return True


def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
              fixed_max: Optional[float] = None, out_dtype: torch.dtype = torch.bfloat16, want_lse: bool = False
              ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``(O, lse)`` for bf16 ``q [B, H, Nq, D]``, ``k [B, H, Nk, D]``, ``v [B, H, Nk, Dv]`` (any strides with a
    contiguous last dimension).  ``O`` is returned as a ``[B, H, Nq, Dv]`` view of a ``[B, Nq, H, Dv]`` buffer, so
    the usual ``o.transpose(1, 2).reshape(B, Nq, H * Dv)`` is free.  ``fixed_max``: an upper bound of
    ``scale * q.k`` known in advance (removes the running-maximum rescaling)."""
    from . import fused as _f
    from . import gemm as _gemm
    b, h, nq, d = q.shape
    nk, dv = k.shape[2], v.shape[3]
    scale = 1.0 / math.sqrt(d) if scale is None else float(scale)
    o = torch.empty((b, nq, h, dv), dtype=out_dtype, device=q.device).transpose(1, 2)
    lse = torch.empty((b * h, nq), dtype=torch.float32, device=q.device) if want_lse else None
    L = _f.lib()
    L.tsp_attn_fwd.restype = _c.c_int
    with _f.on_device(q.device):
        code = L.tsp_attn_fwd(_f._ptr(q), _f._ptr(k), _f._ptr(v), _f._ptr(o), _f._ptr(lse), _c.c_int(b), _c.c_int(h),
                              _c.c_int(nq), _c.c_int(nk), _c.c_int(d), _c.c_int(dv), _strides3(q), _strides3(k),
                              _strides3(v), _strides3(o), _c.c_float(scale),
                              _c.c_float(0.0 if fixed_max is None else float(fixed_max)),
                              _c.c_int(0 if fixed_max is None else 1), _c.c_int(_f._dt(o)),
                              _f._ptr(_gemm._status_word(q.device)), _f._stream())
    _f._check(code, "tsp_attn_fwd")
    _f._count()
    return o, (lse.view(b, h, nq) if want_lse else None)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor] = None,
              dropout_p: float = 0.0) -> torch.Tensor:
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if _TCGEN05 and mask is None and dropout_p == 0.0 and not needs_grad and q.shape[-1] == 64 \
            and flash_eligible(q, k, v):
        return flash_fwd(q, k, v)[0]
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=dropout_p)
