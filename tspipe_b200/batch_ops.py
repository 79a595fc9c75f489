"""Mini-batch / micro-batch containers and the user-overridable scatter/gather pair.

API parity with `tspipe/batch_ops.py`: :class:`Batch` (`:24-149`), :func:`scatter` /
:func:`gather` (`:168-205`), :class:`ScatterGatherFn` (`:208-221`), :class:`BatchQueue` (`:256-297`).
The reference's ``Microbatch`` / ``BatchList`` envelopes (`:224-253`) have no counterpart: a microbatch is identified
by its position in the schedule (``schedule.Op``: batch, view, microbatch), not by a tagged message."""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor

from .utils import pytree as pt

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]


class Batch:
    """A tensor, a tuple of tensors, or any pytree, with uniform access."""

    def __init__(self, value: Any):
        self.value = value
        self.atomic = torch.is_tensor(value)

    @property
    def tensor(self) -> Tensor:
        if not self.atomic:
            raise AttributeError("not atomic batch")
        return self.value

    @property
    def tensors(self) -> Tensors:
        if self.atomic:
            raise AttributeError("batch is atomic")
        return self.value

    @property
    def tensor_or_tensors(self) -> Any:
        return self.value

    def call(self, fn: Callable) -> "Batch":
        return Batch(fn(self.value))

    def __repr__(self) -> str:
        return f"Batch[atomic={self.atomic!r}]({self.value!r})"

    def __iter__(self):
        if self.atomic:
            yield self.value
        else:
            yield from self.value

    def __len__(self) -> int:
        return 1 if self.atomic else len(self.value)

    def __getitem__(self, index):
        if self.atomic:
            if index != 0:
                raise IndexError("atomic batch allows index 0 only")
            return self.value
        return self.value[index]


def check(input: Any) -> None:
    if isinstance(input, tuple):
        for x in input:
            check(x)
        return
    if not isinstance(input, Tensor):
        raise TypeError(f"expected Tensor, but got {input.__class__.__name__}")


def scatter(input: Any, chunks: int) -> List[Batch]:
    """Split a mini-batch into ``chunks`` micro-batches along dim 0 (views, no copy)."""
    if isinstance(input, Tensor):
        parts = input.chunk(chunks)
        if len(parts) != chunks:
            raise ValueError(f"batch of {input.shape[0]} cannot be split into {chunks} micro-batches")
        return [Batch(x) for x in parts]
    return [Batch(x) for x in pt.generic_scatter(input, chunks)]


def gather(outputs: Sequence[Batch]) -> Any:
    """Concatenate micro-batch outputs back into a mini-batch."""
    if outputs[0].atomic:
        return torch.cat([b.tensor for b in outputs]) if len(outputs) > 1 else outputs[0].tensor
    return pt.generic_gather([b.value for b in outputs])


def batch_size(t: Any) -> int:
    if torch.is_tensor(t):
        return t.shape[0]
    return pt.leading_size(t)


@dataclass
class ScatterGatherFn:
    scatter: Callable[[Any, int], List[Batch]]
    gather: Callable[[List[Batch]], Any]
    batch_size: Callable[[Any], int]


defaultScatterGatherFn = ScatterGatherFn(scatter=scatter, gather=gather, batch_size=batch_size)


class BatchQueue:
    """Batch-id allocation, epoch boundaries, and the 'has batch b been fed?' throttle."""

    def __init__(self):
        self.next_id = 1
        self.highest_ready_batch_id = 0
        self.cv = threading.Condition()
        self.running = True
        self.epoch_boundaries: List[int] = []

    def get_new_batch_id(self) -> int:
        with self.cv:
            r = self.next_id
            self.highest_ready_batch_id = max(r, self.highest_ready_batch_id)
            self.next_id += 1
            self.cv.notify_all()
        return r

    def report_epoch_boundary(self) -> None:
        with self.cv:
            self.epoch_boundaries.append(self.next_id - 1)
            self.cv.notify_all()

    def stop(self) -> None:
        with self.cv:
            self.running = False
            self.cv.notify_all()

    def wait_batch(self, batch_id: int, timeout: Optional[float] = None) -> bool:
        """True when ``batch_id`` has been fed; False when feeding has stopped before it."""
        with self.cv:
            while batch_id > self.highest_ready_batch_id and self.running:
                if not self.cv.wait(timeout):
                    return False
            return batch_id <= self.highest_ready_batch_id
