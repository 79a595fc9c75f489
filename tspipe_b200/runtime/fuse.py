"""Peephole fusion of a stage partition's children.

A partition is an ``nn.Sequential`` whose child granularity is part of the user-facing contract
(``model_split`` counts children, checkpoints are keyed by child names), so the modules stay as they
are; only the way the partition *runs* them changes.  :class:`FusedSequential` executes the same
children in order but lets neighbouring ones share a kernel:

* ``BatchNorm -> ReLU``                      one fused normalise + activation pass (``ops.bn.bn_act``);
* ``Conv2d(3, 64, 7, stride 2) -> BatchNorm`` the tcgen05 stem convolution, whose epilogue already produces the
  BatchNorm statistics (``ops.conv.stem_conv``), so the statistics pass over the activation disappears;
* ``Linear`` children (the MLP heads)        the tcgen05 GEMM path of ``ops.linear.linear``, forward and backward.

The reference runs these layers one library call at a time
(`benchmarks/byol/models/resnet_base_network.py`, `tspipe/tspipe.py:553-580` for the child granularity).
"""
from __future__ import annotations

from typing import Any, List

import torch
from torch import nn
from torch.nn.modules.batchnorm import _BatchNorm


class FusedSequential(nn.Sequential):
    """Same children, same parameters and state-dict keys as the ``nn.Sequential`` it replaces."""

    def forward(self, x: Any) -> Any:  # type: ignore[override]
        from ..ops import bn as _bn
        from ..ops import conv as _conv
        from ..ops import linear as _linear
        mods: List[nn.Module] = list(self._modules.values())
        i, n = 0, len(mods)
        while i < n:
            m = mods[i]
            nxt = mods[i + 1] if i + 1 < n else None
            if _conv.is_stem_conv(m) and _conv.eligible(x) and torch.is_autocast_enabled():
                bn_next = isinstance(nxt, _BatchNorm) and nxt.training
                segs = _bn.current_segments() if x.shape[0] % _bn.current_segments() == 0 else 1
                bn_next = bn_next and (segs == _bn.current_segments())
                y, sums = _conv.stem_conv(x, m.weight, want_sums=bn_next, segments=segs)
                if bn_next and _bn.applicable(nxt, y):
                    relu = i + 2 < n and isinstance(mods[i + 2], nn.ReLU)
                    x = _bn.bn_act(nxt, y, relu=relu, sums=sums)
                    i += 3 if relu else 2
                else:
                    x = y
                    i += 1
                continue
            if isinstance(m, _BatchNorm) and isinstance(nxt, nn.ReLU) and isinstance(x, torch.Tensor) \
                    and _bn.applicable(m, x):
                x = _bn.bn_act(m, x, relu=True)
                i += 2
                continue
            if type(m) is nn.Linear and isinstance(x, torch.Tensor):
                x = _linear.linear(x, m.weight, m.bias)
                i += 1
                continue
            x = m(x)
            i += 1
        return x


def fuse_partition(module: nn.Module) -> nn.Module:
    """Switch a plain ``nn.Sequential`` partition to fused execution (in place; no-op for anything else)."""
    if type(module) is nn.Sequential:
        module.__class__ = FusedSequential
    return module
