"""Scaled dot-product attention ``softmax(Q K^T / sqrt(d) + mask) V`` for [B, H, N, D] tensors.

The reference models run it unfused - two batched GEMMs, a softmax and a dropout
(timm ``Attention`` in `benchmarks/moco-v3/vits.py`, HF ``BertSelfAttention`` in
`benchmarks/distilbert/bert.py`).  Here it is one fused call; ``mask`` is an additive or boolean
key-padding mask broadcastable to [B, 1, 1, N] / [B, H, N, N].
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor] = None,
              dropout_p: float = 0.0) -> torch.Tensor:
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=dropout_p)
