"""Flat parameter / gradient storage for one partition.

The reference keeps every parameter version as a Python list of cloned tensors
(`tspipe/gpu_context.py:81-143`) and rewrites the live module with one ``copy_`` per
tensor (`tspipe/gpu_task.py:720-724`).  Here each partition's parameters live in ONE
contiguous fp32 buffer (and their gradients in another); the module's ``Parameter``s are
views into it.  One buffer means one launch for the optimizer, one for the momentum-teacher
update, one ``memset`` for ``zero_grad``, a contiguous range to reduce-scatter across
pipeline replicas and a single base pointer to publish to peer GPUs.

The schedule orders every teacher forward of batch ``b+1`` between ``OPT(b-1)`` and
``OPT(b)`` on its device, so the in-place update needs no second copy of the parameters.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
from torch import nn

ALIGN = 64          # elements; 256 B for fp32 so every tensor starts on a vector-load boundary


def _is_channels_last(t: torch.Tensor) -> bool:
    return t.dim() == 4 and not t.is_contiguous() and t.is_contiguous(memory_format=torch.channels_last)


class FlatParams:
    """Flatten ``params`` into one buffer; keeps shapes, offsets and memory formats."""

    def __init__(self, params: Sequence[nn.Parameter], device: torch.device, with_grad: bool,
                 dtype: torch.dtype = torch.float32, pad_to: int = 1):
        self.params: List[nn.Parameter] = list(params)
        self.device, self.dtype = device, dtype
        self.offsets: List[int] = []
        self.numels: List[int] = []
        off = 0
        for p in self.params:
            self.offsets.append(off)
            self.numels.append(p.numel())
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.total = max(off, ALIGN)
        if pad_to > 1:
            unit = ALIGN * pad_to
            self.total = (self.total + unit - 1) // unit * unit
        self.data = torch.zeros(self.total, dtype=dtype, device=device)
        self.grad = torch.zeros(self.total, dtype=dtype, device=device) if with_grad else None
        self._bind()

    def _view(self, flat: torch.Tensor, i: int, like: torch.Tensor) -> torch.Tensor:
        seg = flat[self.offsets[i]: self.offsets[i] + self.numels[i]]
        if _is_channels_last(like):
            n, c, h, w = like.shape
            return seg.view(n, h, w, c).permute(0, 3, 1, 2)
        return seg.view(like.shape)

    def _bind(self) -> None:
        with torch.no_grad():
            for i, p in enumerate(self.params):
                v = self._view(self.data, i, p.data)
                v.copy_(p.data)
                p.data = v
                if self.grad is not None and p.requires_grad:
                    p.grad = self._view(self.grad, i, p.data)

    def rebind_data(self, flat: torch.Tensor) -> None:
        """Point the parameters at another buffer of the same layout (e.g. symmetric memory)."""
        assert flat.numel() == self.total and flat.dtype == self.dtype
        flat.copy_(self.data)
        self.data = flat
        for i, p in enumerate(self.params):
            p.data = self._view(flat, i, p.data)

    def zero_grad(self) -> None:
        if self.grad is None:
            return
        self.grad.zero_()
        for i, p in enumerate(self.params):      # autograd may have replaced .grad; re-attach the view
            if p.requires_grad and (p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + 4 * self.offsets[i]):
                p.grad = self._view(self.grad, i, p.data)

    def collect_stray_grads(self) -> None:
        """Fold gradients that autograd placed outside the flat buffer back into it."""
        if self.grad is None:
            return
        esz = self.grad.element_size()
        for i, p in enumerate(self.params):
            if p.grad is None or not p.requires_grad:
                continue
            if p.grad.data_ptr() != self.grad.data_ptr() + esz * self.offsets[i]:
                v = self._view(self.grad, i, p.data)
                v.add_(p.grad)
                p.grad = v

    # -- tables for the multi-tensor kernels -------------------------------------------------------
    def segment_table(self) -> Tuple[torch.Tensor, torch.Tensor]:
        off = torch.tensor(self.offsets, dtype=torch.int64, device=self.device)
        num = torch.tensor(self.numels, dtype=torch.int64, device=self.device)
        return off, num

    def shapes(self) -> List[Tuple[int, ...]]:
        return [tuple(p.shape) for p in self.params]


def corresponding_prefix(student: FlatParams, teacher: FlatParams) -> bool:
    """True when the teacher layout equals a prefix of the student layout (same split for
    both nets; the student may carry extra predictor parameters at the end)."""
    nt = len(teacher.params)
    if nt > len(student.params):
        return False
    return (student.offsets[:nt] == teacher.offsets and student.numels[:nt] == teacher.numels
            and all(_is_channels_last(a.data) == _is_channels_last(b.data)
                    for a, b in zip(student.params[:nt], teacher.params)))
