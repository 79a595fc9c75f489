"""Failure detection: heartbeats and death notices through the rendezvous store.

The reference has none - no heartbeats, no timeouts on RPC or NCCL, a crashed worker leaves the others
blocked in ``queue.get()`` / ``dist.recv`` (`tspipe/gpu_worker.py:119,300,590-591`).  Here every rank

* publishes ``hb/<rank> = (wall time, ops executed, busy)`` every ``runtime.heartbeat_s`` seconds (``busy``:
  the executor is inside a schedule operation right now),
* publishes ``dead/<rank> = reason`` when its executor dies with an exception,
* and watches the other ranks: a death notice, a heartbeat older than ``runtime.timeout_s`` (the process is
  gone), or a rank that stays busy on the same operation count for ``runtime.timeout_s`` (the process lives,
  its heartbeat thread keeps beating, but the executor is stuck in a collective or a stream wait) marks the
  local engine as failed with a :class:`PeerFailure`, which the feeding thread raises from the next
  ``feed`` / ``flush`` / ``stop`` instead of waiting forever.  Device-side waits are bounded separately
  (status words written by the kernels, see ``mbar_wait`` in ``csrc/gemm_tcgen05.cu`` and ``tsp_signal_wait``
  in ``csrc/peer.cu``).

Faults are detected on the host only; nothing here touches a GPU.
"""
from __future__ import annotations

import pickle
import threading
import time
from typing import Callable, Dict, Optional


class PeerFailure(RuntimeError):
    pass


class Watchdog:
    def __init__(self, store, rank: int, world: int, heartbeat_s: float, timeout_s: float,
                 progress: Callable[[], int], on_failure: Callable[[BaseException], None],
                 clock: Callable[[], float] = time.time, busy: Optional[Callable[[], bool]] = None):
        self.store, self.rank, self.world = store, rank, world
        self.heartbeat_s, self.timeout_s = float(heartbeat_s), float(timeout_s)
        self.progress, self.on_failure, self.clock = progress, on_failure, clock
        self.busy = busy if busy is not None else (lambda: False)
        self._last_ops: Dict[int, tuple] = {}        # peer -> (ops, local time at which that count was first seen)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.failed: Optional[PeerFailure] = None
        self._first_seen: Dict[int, float] = {}

    def start(self) -> None:
        self.beat()
        self._thread = threading.Thread(target=self._run, name=f"tspipe-watchdog-{self.rank}", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        try:
            self.store.set(f"bye/{self.rank}", b"1")
        except Exception:
            pass

    def halt(self) -> None:
        """Stop beating and watching without the orderly good-bye (the executor died with an error)."""
        self._stop.set()

    def beat(self) -> None:
        self.store.set(f"hb/{self.rank}", pickle.dumps((self.clock(), int(self.progress()), bool(self.busy()))))

    def announce_death(self, reason: str) -> None:
        try:
            self.store.set(f"dead/{self.rank}", reason.encode()[:2000])
        except Exception:
            pass

    def check_once(self) -> Optional[PeerFailure]:
        """One sweep over the peers (also callable directly from tests)."""
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check([f"dead/{r}"]):
                why = self.store.get(f"dead/{r}").decode(errors="replace")
                return PeerFailure(f"rank {r} failed: {why}")
            if self.store.check([f"bye/{r}"]):
                continue
            if self.store.check([f"hb/{r}"]):
                rec = pickle.loads(self.store.get(f"hb/{r}"))
                t, ops = rec[0], rec[1]
                peer_busy = bool(rec[2]) if len(rec) > 2 else False
                if now - t > self.timeout_s:
                    return PeerFailure(f"rank {r} has been silent for {now - t:.1f} s (limit {self.timeout_s} s)")
                seen = self._last_ops.get(r)
                if seen is None or seen[0] != ops or not peer_busy:
                    self._last_ops[r] = (ops, now)
                elif now - seen[1] > self.timeout_s:
                    return PeerFailure(f"rank {r} is stalled: busy on operation {ops} for {now - seen[1]:.1f} s "
                                       f"(limit {self.timeout_s} s)")
            else:
                first = self._first_seen.setdefault(r, now)
                if now - first > self.timeout_s:
                    return PeerFailure(f"rank {r} never reported within {self.timeout_s} s")
        return None

    def _run(self) -> None:
        while not self._stop.wait(self.heartbeat_s):
            try:
                self.beat()
                f = self.check_once()
            except Exception:       # store gone: the job is shutting down
                return
            if f is not None:
                self.failed = f
                self.on_failure(f)
                return
