"""Scalars, throughput and the final ``model.pth`` of a training run.

The reference applications log ``loss`` / ``learning_rate`` / ``momentum`` to TensorBoard
(`benchmarks/byol/trainer.py:29,98,262-273`, `benchmarks/moco-v3/main.py:281,432,472`,
`benchmarks/soft_target/train_kd.py:233,410`) and end with ``model.pth`` holding the three keys
``online_network_state_dict`` / ``target_network_state_dict`` / ``optimizer_state_dict``
(`benchmarks/byol/trainer.py:151-157,279`).  :class:`RunLog` does both for the applications here: scalars go to a
TensorBoard event file when the ``tensorboard`` package is importable and always to ``scalars.csv`` next to it;
:class:`ThroughputMeter` is the runtime's samples-per-second counter (:attr:`tspipe_b200.TSPipe.meter`).
"""
from __future__ import annotations

import os
import time
from typing import Any, Dict, Optional

import torch


class ThroughputMeter:
    """Samples per second as seen by the feeder: overall since the first batch, and over a sliding window."""

    def __init__(self, window: int = 20):
        self.window = max(int(window), 1)
        self.samples = 0
        self.batches = 0
        self._t0: Optional[float] = None
        self._marks = []          # (time, samples) of the last `window` batches

    def add(self, n_samples: int, now: Optional[float] = None) -> None:
        now = time.perf_counter() if now is None else now
        if self._t0 is None:
            self._t0 = now
            self._marks.append((now, 0))
        self.samples += int(n_samples)
        self.batches += 1
        self._marks.append((now, self.samples))
        if len(self._marks) > self.window + 1:
            self._marks.pop(0)

    def overall(self, now: Optional[float] = None) -> float:
        if self._t0 is None:
            return 0.0
        now = time.perf_counter() if now is None else now
        dt = now - self._t0
        return self.samples / dt if dt > 0 else 0.0

    def recent(self) -> float:
        """Rate over the last ``window`` batches (first batch of the window excluded: its time is the origin)."""
        if len(self._marks) < 2:
            return 0.0
        (t0, s0), (t1, s1) = self._marks[0], self._marks[-1]
        return (s1 - s0) / (t1 - t0) if t1 > t0 else 0.0


class RunLog:
    def __init__(self, log_dir: str, enabled: bool = True, tensorboard: bool = True):
        self.log_dir, self.enabled = log_dir, bool(enabled)
        self._csv = None
        self._tb = None
        if not self.enabled:
            return
        os.makedirs(log_dir, exist_ok=True)
        self._csv = open(os.path.join(log_dir, "scalars.csv"), "a", buffering=1)
        if self._csv.tell() == 0:
            self._csv.write("wall_time,step,tag,value\n")
        if tensorboard:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self._tb = SummaryWriter(log_dir=log_dir)
            except Exception:          # package missing or broken: the CSV is the record
                self._tb = None

    def scalar(self, tag: str, value: float, step: int) -> None:
        if not self.enabled:
            return
        value = float(value)
        self._csv.write(f"{time.time():.3f},{int(step)},{tag},{value:.8g}\n")
        if self._tb is not None:
            self._tb.add_scalar(tag, value, global_step=int(step))

    def save_final(self, tsp: Any, optimizer: Optional[torch.optim.Optimizer], path: Optional[str] = None) -> Optional[str]:
        """After ``tsp.stop()``: ``model.pth`` with the whole student and teacher state dicts (the per-partition
        dicts of :meth:`TSPipe.state_dicts` joined in partition order) and the optimizer's."""
        if not self.enabled:
            return None
        online, target = tsp.state_dicts()
        if not online and not target:
            return None
        path = path or os.path.join(self.log_dir, "model.pth")
        torch.save({"online_network_state_dict": join_partitions(online),
                    "target_network_state_dict": join_partitions(target),
                    "optimizer_state_dict": optimizer.state_dict() if optimizer is not None else {}}, path)
        return path

    def close(self) -> None:
        if self._tb is not None:
            self._tb.close()
            self._tb = None
        if self._csv is not None:
            self._csv.close()
            self._csv = None


def join_partitions(parts: Dict[int, Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for idx in sorted(parts):
        for k, v in parts[idx].items():
            if k in out:
                raise KeyError(f"state-dict key {k!r} appears in two partitions")
            out[k] = v
    return out
