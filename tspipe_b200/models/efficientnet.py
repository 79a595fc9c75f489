"""EfficientNet (B0-B3 scaling) as a :class:`~tspipe_b200.model_base.SequentialableModel`.

The soft-target benchmark of the reference can distil into / from EfficientNets
(`benchmarks/soft_target/models/efficient_net.py:38-149,408-445`, helpers in `efficient_net_utils.py`: swish,
drop-connect, "same" padding).  This is a compact re-implementation with the same block structure: stem conv-BN-
swish, MBConv blocks (expand 1x1, depthwise kxk, squeeze-excite, project 1x1, drop-connect + identity skip), head
conv-BN-swish, pool, dropout, classifier.  ``to_sequential`` yields one child per stem op / block / head op, with
each block's drop-connect rate scaled by its depth (`efficient_net.py:426-431`).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import List, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..model_base import FlattenWrapper, SequentialableModel

# (expand_ratio, channels, repeats, stride, kernel)
_B0: List[Tuple[int, int, int, int, int]] = [(1, 16, 1, 1, 3), (6, 24, 2, 2, 3), (6, 40, 2, 2, 5), (6, 80, 3, 2, 3),
                                             (6, 112, 3, 1, 5), (6, 192, 4, 2, 5), (6, 320, 1, 1, 3)]
_SCALING = {"efficientnet-b0": (1.0, 1.0, 0.2), "efficientnet-b1": (1.0, 1.1, 0.2),
            "efficientnet-b2": (1.1, 1.2, 0.3), "efficientnet-b3": (1.2, 1.4, 0.3),
            "efficientnet-tiny-test": (0.25, 0.34, 0.0)}


def _round_filters(c: int, width: float, divisor: int = 8) -> int:
    c *= width
    new = max(divisor, int(c + divisor / 2) // divisor * divisor)
    if new < 0.9 * c:
        new += divisor
    return int(new)


def drop_connect(x: torch.Tensor, p: float, training: bool) -> torch.Tensor:
    """Drop whole samples of a residual branch with probability ``p`` (stochastic depth)."""
    if not training or p <= 0:
        return x
    keep = 1.0 - p
    mask = torch.floor(keep + torch.rand((x.shape[0], 1, 1, 1), dtype=x.dtype, device=x.device))
    return x / keep * mask


class MBConv(nn.Module):
    def __init__(self, cin: int, cout: int, expand: int, stride: int, kernel: int, se_ratio: float = 0.25,
                 drop_connect_rate: float = 0.0, eps: float = 1e-3, momentum: float = 0.01):
        super().__init__()
        mid = cin * expand
        self.expand = None
        if expand != 1:
            self.expand = nn.Sequential(nn.Conv2d(cin, mid, 1, bias=False), nn.BatchNorm2d(mid, eps, momentum))
        self.depthwise = nn.Sequential(nn.Conv2d(mid, mid, kernel, stride, kernel // 2, groups=mid, bias=False),
                                       nn.BatchNorm2d(mid, eps, momentum))
        sq = max(1, int(cin * se_ratio))
        self.se_reduce, self.se_expand = nn.Conv2d(mid, sq, 1), nn.Conv2d(sq, mid, 1)
        self.project = nn.Sequential(nn.Conv2d(mid, cout, 1, bias=False), nn.BatchNorm2d(cout, eps, momentum))
        self.skip = stride == 1 and cin == cout
        self.drop_connect_rate = drop_connect_rate

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = x
        if self.expand is not None:
            h = F.silu(self.expand(h))
        h = F.silu(self.depthwise(h))
        s = self.se_expand(F.silu(self.se_reduce(h.mean((2, 3), keepdim=True))))
        h = self.project(torch.sigmoid(s) * h)
        if self.skip:
            h = drop_connect(h, self.drop_connect_rate, self.training) + x
        return h


class EfficientNet(SequentialableModel):
    def __init__(self, name: str = "efficientnet-b0", num_classes: int = 1000, drop_connect_rate: float = 0.2):
        super().__init__()
        width, depth, dropout = _SCALING[name]
        stem = _round_filters(32, width)
        self.stem = nn.Sequential(nn.Conv2d(3, stem, 3, 2, 1, bias=False), nn.BatchNorm2d(stem, 1e-3, 0.01), nn.SiLU())
        blocks: List[MBConv] = []
        cin = stem
        cfg = [(e, _round_filters(c, width), int(math.ceil(r * depth)), s, k) for e, c, r, s, k in _B0]
        total = sum(r for _, _, r, _, _ in cfg)
        for e, c, r, s, k in cfg:
            for i in range(r):
                rate = drop_connect_rate * len(blocks) / total
                blocks.append(MBConv(cin, c, e, s if i == 0 else 1, k, drop_connect_rate=rate))
                cin = c
        self.blocks = nn.ModuleList(blocks)
        head = _round_filters(1280, width)
        self.head = nn.Sequential(nn.Conv2d(cin, head, 1, bias=False), nn.BatchNorm2d(head, 1e-3, 0.01), nn.SiLU())
        self.pool, self.flatten = nn.AdaptiveAvgPool2d(1), FlattenWrapper(1)
        self.dropout, self.fc = nn.Dropout(dropout), nn.Linear(head, num_classes)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.stem(x)
        for b in self.blocks:
            x = b(x)
        return self.fc(self.dropout(self.flatten(self.pool(self.head(x)))))

    def to_sequential(self) -> nn.Sequential:
        ch = OrderedDict()
        for i, m in enumerate(self.stem):
            ch[f"stem{i}"] = m
        for i, b in enumerate(self.blocks):
            ch[f"block{i}"] = b
        for i, m in enumerate(self.head):
            ch[f"head{i}"] = m
        ch["pool"], ch["flatten"], ch["dropout"], ch["fc"] = self.pool, self.flatten, self.dropout, self.fc
        return nn.Sequential(ch)
