"""Event trace in the reference's CSV schema (`tspipe/profiler.py:25-150`).

``with TSPipeProfiler(filename='profile_out.csv') as prof:`` collects rows
``timestamp_ms, batch_idx, view_idx, ubatch_idx, is_target, src_partition, dst_partition, op`` where
``op`` is an operation name on entry and ``<name>_finish`` on exit (the reference's ``Operation`` context
manager, `:117-150`), and flushes them to the file from a writer thread every 250 ms (`:68-88`).

Differences: the reference's timestamps are host wall-clock and only meaningful because every task ends
in a device synchronisation.  Here the executor never synchronises, so each ``Operation`` additionally
records a pair of CUDA events on its stream; :meth:`TSPipeProfiler.device_times` resolves them to
per-operation device milliseconds (column ``device_ms`` of ``<filename>.device.csv``), and NVTX ranges are
pushed when ``nvtx=True``.  In launcher mode every rank writes its own file (``.rank<r>`` suffix) instead of
funnelling rows to rank 0 over RPC (`tspipe/profiler.py:95-114`).
"""
from __future__ import annotations

import csv
import os
import queue
import threading
import time
from typing import Any, List, Optional, Tuple

import torch

_active: Optional["TSPipeProfiler"] = None


def _now_ms() -> float:
    return time.time() * 1000.0


class Operation:
    """Context manager logging ``op`` and ``op_finish`` rows (plus device events on CUDA)."""

    def __init__(self, op: str, batch_idx: int = 0, view_idx: int = 0, ubatch_idx: int = 0, is_target: bool = False,
                 src_partition: Optional[int] = None, dst_partition: Optional[int] = None,
                 profiler: Optional["TSPipeProfiler"] = None):
        self.row = [batch_idx, view_idx, ubatch_idx, int(bool(is_target)), src_partition, dst_partition]
        self.op = op
        self.prof = profiler if profiler is not None else _active
        self.ev = None

    def __enter__(self) -> "Operation":
        p = self.prof
        if p is None:
            return self
        p.log([_now_ms()] + self.row + [self.op])
        if p.cuda_events and torch.cuda.is_available():
            self.ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self.ev[0].record()
        if p.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(f"{self.op} b{self.row[0]} v{self.row[1]} u{self.row[2]}")
        return self

    def __exit__(self, *exc) -> None:
        p = self.prof
        if p is None:
            return
        if p.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        if self.ev is not None:
            self.ev[1].record()
            p.device_events.append((self.op, tuple(self.row), self.ev))
        p.log([_now_ms()] + self.row + [self.op + "_finish"])


def profile_semantic(batch_idx: int, view_idx: int, ubatch_idx: int, is_target: bool, src_partition, dst_partition,
                     op: str) -> None:
    """One-off row (`tspipe/profiler.py:58-60`)."""
    if _active is not None:
        _active.log([_now_ms(), batch_idx, view_idx, ubatch_idx, int(bool(is_target)), src_partition, dst_partition, op])


class TSPipeProfiler:
    HEADER = ["timestamp_ms", "batch_idx", "view_idx", "ubatch_idx", "is_target", "src_partition", "dst_partition", "op"]

    def __init__(self, filename: str = "profile_out.csv", cuda_events: bool = True, nvtx: bool = False,
                 flush_every_s: float = 0.25):
        rank = os.environ.get("RANK")
        self.filename = filename if rank in (None, "0") else f"{filename}.rank{rank}"
        self.cuda_events, self.nvtx, self.flush_every_s = cuda_events, nvtx, flush_every_s
        self.q: "queue.Queue[List[Any]]" = queue.Queue()
        self.device_events: List[Tuple[str, Tuple, Tuple]] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    # -- context manager ---------------------------------------------------------------------------
    def __enter__(self) -> "TSPipeProfiler":
        global _active
        d = os.path.dirname(self.filename)
        if d:
            os.makedirs(d, exist_ok=True)
        self._fh = open(self.filename, "w", newline="")
        self._writer = csv.writer(self._fh)
        self._writer.writerow(self.HEADER)
        self._thread = threading.Thread(target=self._run, name="tspipe-profiler", daemon=True)
        self._thread.start()
        _active = self
        return self

    def __exit__(self, *exc) -> None:
        global _active
        _active = None
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        self._drain()
        self._fh.close()
        if self.device_events:
            self.write_device_times()

    # -- logging -------------------------------------------------------------------------------------
    def log(self, row: List[Any]) -> None:
        self.q.put(row)

    def operation(self, op: str, batch_idx: int, view_idx: int, ubatch_idx: int, is_target: bool,
                  partition: Optional[int]) -> Operation:
        return Operation(op, batch_idx, view_idx, ubatch_idx, is_target, None, partition, profiler=self)

    def _drain(self) -> None:
        while True:
            try:
                self._writer.writerow(self.q.get_nowait())
            except queue.Empty:
                break
        self._fh.flush()

    def _run(self) -> None:
        while not self._stop.wait(self.flush_every_s):
            self._drain()

    # -- device timing -------------------------------------------------------------------------------
    def device_times(self) -> List[Tuple[str, Tuple, float]]:
        """``(op, (batch, view, ubatch, is_target, src, dst), device_ms)`` for every finished operation."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = []
        for op, row, (e0, e1) in self.device_events:
            try:
                out.append((op, row, e0.elapsed_time(e1)))
            except RuntimeError:
                pass
        return out

    def write_device_times(self) -> str:
        path = self.filename + ".device.csv"
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["op"] + self.HEADER[1:7] + ["device_ms"])
            for op, row, ms in self.device_times():
                w.writerow([op] + list(row) + [f"{ms:.4f}"])
        return path
