"""Data-loading helpers (`tspipe/dataloader.py:11-87`).

``FastDataLoader``: a ``DataLoader`` whose worker processes survive across epochs (the reference
re-implements this with a repeat sampler; PyTorch has ``persistent_workers`` for it).
``SuperFastDataLoader``: the loader itself runs in a child process and hands batches over a queue, so
that collation never competes with the feeding thread.
``DummyInputGenerator``: two fixed random views in shared / pinned memory, length 30, for
throughput-only runs.
"""
from __future__ import annotations

from typing import Any, Iterator

import torch
from torch.utils.data import DataLoader


class FastDataLoader(DataLoader):
    def __init__(self, *args, **kwargs):
        if kwargs.get("num_workers", 0) > 0:
            kwargs.setdefault("persistent_workers", True)
        super().__init__(*args, **kwargs)


_EPOCH_END, _ALL_DONE = "__epoch_end__", "__all_done__"


def _producer(loader_args, loader_kwargs, q, epochs, done):
    loader = DataLoader(*loader_args, **loader_kwargs)
    for _ in range(epochs):
        for batch in loader:
            q.put(batch)
        q.put(_EPOCH_END)
    q.put(_ALL_DONE)
    done.wait(600)          # shared-memory tensors in flight die with this process: leave only when told


class SuperFastDataLoader:
    """Iterate a ``DataLoader`` that lives in a child process."""

    def __init__(self, *args, epochs: int = 1, prefetch: int = 4, **kwargs):
        self.args, self.kwargs, self.epochs, self.prefetch = args, kwargs, epochs, prefetch
        self._len = len(DataLoader(*args, **{**kwargs, "num_workers": 0}))
        self._q = None
        self._proc = None

    def __len__(self) -> int:
        return self._len

    def _start(self) -> None:
        ctx = torch.multiprocessing.get_context("spawn")
        self._q = ctx.Queue(self.prefetch)
        self._done = ctx.Event()
        self._proc = ctx.Process(target=_producer, args=(self.args, self.kwargs, self._q, self.epochs, self._done),
                                 daemon=True)
        self._proc.start()

    def __iter__(self) -> Iterator[Any]:
        if self._proc is None:
            self._start()
        while True:
            item = self._q.get()
            if isinstance(item, str) and item == _ALL_DONE:
                self._done.set()
                return
            if isinstance(item, str) and item == _EPOCH_END:
                return
            yield item


class DummyInputGenerator:
    """``((view_1, view_2), 0)`` thirty times per epoch; the same two tensors every time."""

    def __init__(self, batch_size: int, input_shape: int = 224, length: int = 30, pin: bool = False,
                 channels: int = 3, dtype: torch.dtype = torch.float32):
        g = torch.Generator().manual_seed(0)
        shape = (batch_size, channels, input_shape, input_shape)
        self.v1 = torch.randn(shape, generator=g).to(dtype)
        self.v2 = torch.randn(shape, generator=g).to(dtype)
        if pin and torch.cuda.is_available():
            self.v1, self.v2 = self.v1.pin_memory(), self.v2.pin_memory()
        else:
            self.v1.share_memory_()
            self.v2.share_memory_()
        self.length = length

    def __len__(self) -> int:
        return self.length

    def __iter__(self):
        for _ in range(self.length):
            yield (self.v1, self.v2), 0
