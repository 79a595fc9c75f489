"""Precision wrapper for the reference arm's bf16 line (``run_reference.py --ref-dtype bf16``).

The reference trains in fp32 only.  To give it the compute precision of the own arm without touching its sources,
every child of the ``nn.Sequential`` models handed to the stock ``tspipe.TSPipe`` is wrapped in a module whose
forward runs the child under ``torch.autocast(bfloat16)``; parameters stay fp32 (what ``torch.autocast`` training
normally looks like).  The class lives in an importable module because the reference pickles its model partitions
to spawned worker processes (`tspipe/tspipe.py:224`, `tspipe/gpu_worker.py:596-600`).
"""
from collections import OrderedDict

import torch
from torch import nn


class AutocastChild(nn.Module):
    def __init__(self, inner: nn.Module):
        super().__init__()
        self.inner = inner

    def forward(self, *args, **kwargs):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return self.inner(*args, **kwargs)


def autocast_children(seq: nn.Sequential) -> nn.Sequential:
    return nn.Sequential(OrderedDict((name, AutocastChild(m)) for name, m in seq.named_children()))
