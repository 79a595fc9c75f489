"""Device-side signals between the ranks of a group: counters in peer-mapped memory, waited on with a time limit.

Each rank owns a pad of ``len(group)`` int32 words; rank ``i`` announces phase ``v`` by storing ``v`` into word ``i`` of
EVERY rank's pad (``csrc/peer.cu: tsp_signal_arrive``, a tiny kernel on the caller's stream, so everything enqueued
before it is visible to a peer that sees the value), and waits for phase ``v`` with a kernel that spins until all words
of its own pad have reached ``v`` (``tsp_signal_wait``).  The spin is bounded: after ``limit_ms`` the kernel writes an
error code into a status word and returns, the stream carries on, and :meth:`SignalPad.check` raises on the host.
Phases are increasing counters, so a pad never needs resetting.

This replaces stream-ordered tiny NCCL collectives as the ordering primitive of the fused data-parallel kernels
(the reference has no counterpart: no data parallelism in its runtime, host-synchronised everywhere,
`tspipe/communicator.py:631-676`).  Every rank runs on its own GPU: a waiting kernel never shares a GPU with the
kernel it waits for.
"""
from __future__ import annotations

import ctypes as _c
from typing import Sequence

import torch

from . import peer


class SignalTimeout(RuntimeError):
    pass


class SignalPad:
    WAIT_CODE = 11

    def __init__(self, group, group_ranks: Sequence[int], self_index: int, device: torch.device,
                 limit_ms: int = 20000):
        from ..ops import fused
        self.n, self.idx, self.device, self.limit_ms = len(group_ranks), int(self_index), device, int(limit_ms)
        assert 1 <= self.n <= 8
        self.pad = torch.zeros(8, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._views = peer.exchange(self.pad, group, group_ranks)          # keeps the peers' mappings
        self._table = peer.pointer_table(self._views)
        L = fused.lib()
        L.tsp_signal_arrive.restype = _c.c_int
        L.tsp_signal_wait.restype = _c.c_int
        self._lib = L

    def arrive(self, value: int) -> None:
        from ..ops import fused
        with torch.cuda.device(self.device):
            fused._check(self._lib.tsp_signal_arrive(self._table, _c.c_int(self.n), _c.c_int(self.idx), _c.c_int(value),
                                                     fused._stream()), "tsp_signal_arrive")
        fused._count()

    def wait(self, value: int, limit_ms: int = 0) -> None:
        from ..ops import fused
        with torch.cuda.device(self.device):
            fused._check(self._lib.tsp_signal_wait(fused._ptr(self.pad), _c.c_int(self.n), _c.c_int(value),
                                                   _c.c_int(limit_ms or self.limit_ms), fused._ptr(self.status),
                                                   _c.c_int(self.WAIT_CODE), fused._stream()), "tsp_signal_wait")
        fused._count()

    def timed_out(self) -> bool:
        """Synchronising read of the status word (non-zero = a wait gave up); clears it."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
        return code != 0

    def check(self) -> None:
        if self.timed_out():
            raise SignalTimeout(f"a peer of rank index {self.idx} did not signal within {self.limit_ms} ms")
