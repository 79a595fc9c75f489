"""Linear layers: ``y = x @ W^T + b``.

On CUDA under bf16 compute, layers whose shapes fit the tile constraints (feature counts multiples of 64, at least
128 rows) run on the hand-written tcgen05 / TMEM / TMA kernels - forward on the CTA-pair GEMM with the bias in its
epilogue, both backward products on the implicit-GEMM kernels (:mod:`tspipe_b200.ops.gemm`).  Everything else
(CPU, fp32 compute, odd shapes) goes to the library GEMM.  Reference call sites: every ``nn.Linear`` of
`benchmarks/moco-v3/vits.py`, `benchmarks/distilbert/bert.py:104-266`, `benchmarks/byol/models/mlp_head.py:4-26`.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

import os

_USE_TCGEN05 = os.environ.get("TSPIPE_LINEAR", "tcgen05") != "library"      # TSPIPE_LINEAR=library: A/B runs


def set_tcgen05(flag: bool) -> None:
    """Route eligible linears through the tcgen05 kernels (default) or always through the library."""
    global _USE_TCGEN05
    _USE_TCGEN05 = bool(flag)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if _USE_TCGEN05 and x.is_cuda:
        from . import gemm
        if gemm.eligible(x, weight):
            return gemm.linear(x, weight, bias)
    return F.linear(x, weight, bias)
