"""Linear layers: ``y = x @ W^T + b``.

On CUDA with bf16 operands whose shapes fit the tile constraints the product runs on the hand-written
tcgen05 / TMEM / TMA GEMM of ``csrc/gemm_tcgen05.cu`` (:mod:`tspipe_b200.ops.gemm`), forward and both
backward products; everything else goes to the library GEMM.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

_USE_TCGEN05 = False


def set_tcgen05(flag: bool) -> None:
    """Route eligible linears through the tcgen05 kernel (off by default)."""
    global _USE_TCGEN05
    _USE_TCGEN05 = bool(flag)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if _USE_TCGEN05 and x.is_cuda:
        from . import gemm
        if gemm.eligible(x, weight):
            return gemm.linear(x, weight, bias)
    return F.linear(x, weight, bias)
