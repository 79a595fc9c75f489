"""Toy MLPs for the CPU correctness configuration (soft-target KD on 32x32x3 inputs)."""
from __future__ import annotations

from collections import OrderedDict
from typing import Sequence

from torch import nn


def mlp_sequential(widths: Sequence[int], batch_norm: bool = False) -> nn.Sequential:
    """``Flatten`` then Linear(+BN)+ReLU blocks; each block is one child so that it can be cut
    anywhere.  ``widths = [in, h1, ..., out]``."""
    layers = OrderedDict()
    layers["flatten"] = nn.Flatten()
    n = len(widths) - 1
    for i in range(n):
        block = [nn.Linear(widths[i], widths[i + 1])]
        if i < n - 1:
            if batch_norm:
                block.append(nn.BatchNorm1d(widths[i + 1]))
            block.append(nn.ReLU())
        layers[f"fc{i}"] = nn.Sequential(*block) if len(block) > 1 else block[0]
    return nn.Sequential(layers)


def toy_teacher() -> nn.Sequential:
    """8 linear layers 3072 -> 1024 -> ... -> 10."""
    return mlp_sequential([3072, 1024, 1024, 512, 512, 256, 256, 128, 10])


def toy_student() -> nn.Sequential:
    """4 linear layers 3072 -> 512 -> ... -> 10."""
    return mlp_sequential([3072, 512, 256, 128, 10])
