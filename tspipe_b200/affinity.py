"""CPU pinning for worker processes.

The reference parses ``nvidia-smi topo -m`` and calls ``taskset`` (`tspipe/affinity_manager.py:
10-84`): each GPU worker gets up to four exclusive cores, the scheduler the rest.  This
version needs neither binary: it partitions the cores the process is allowed to run on
(``os.sched_getaffinity``) and, when NVML is importable, prefers the cores NVML reports as
local to the GPU.  It is a no-op where the platform has no affinity API, and can be turned off
with ``TSPIPE_NO_AFFINITY=1``.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Set


class AffinityManager:
    CORES_PER_WORKER = 4

    @staticmethod
    def allowed_cores() -> List[int]:
        try:
            return sorted(os.sched_getaffinity(0))
        except AttributeError:
            return list(range(os.cpu_count() or 1))

    @staticmethod
    def gpu_local_cores(gpu_index: int, nvml=None) -> Optional[Set[int]]:
        """Cores NVML lists as close to ``gpu_index`` (None when NVML is not usable).  ``nvml`` may be a
        stand-in object with the three NVML calls used here."""
        try:
            if nvml is None:
                import pynvml as nvml  # type: ignore
                nvml.nvmlInit()
            h = nvml.nvmlDeviceGetHandleByIndex(gpu_index)
            n_words = (max(os.cpu_count() or 64, 64) + 63) // 64
            mask = nvml.nvmlDeviceGetCpuAffinity(h, n_words)
            cores = {w * 64 + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
            return cores or None
        except Exception:
            return None

    @classmethod
    def plan(cls, n_workers: int, allowed: Optional[Sequence[int]] = None,
             local: Optional[Sequence[Optional[Set[int]]]] = None) -> List[List[int]]:
        """Disjoint core sets, one per worker (at most ``CORES_PER_WORKER`` each); whatever is left is
        for the feeding process."""
        allowed = list(allowed if allowed is not None else cls.allowed_cores())
        per = max(1, min(cls.CORES_PER_WORKER, len(allowed) // max(n_workers + 1, 1)))
        free = list(allowed)
        out: List[List[int]] = [[] for _ in range(n_workers)]
        for w in range(n_workers):                 # first the cores that are local to each worker's GPU
            if local and local[w]:
                for c in [c for c in free if c in local[w]][:per]:
                    free.remove(c)
                    out[w].append(c)
        for w in range(n_workers):                 # then fill up from whatever is left
            while len(out[w]) < per and free:
                out[w].append(free.pop(0))
            out[w].sort()
        return out

    @classmethod
    def apply_for_worker(cls, local_index: int, n_workers: int) -> Optional[List[int]]:
        if os.environ.get("TSPIPE_NO_AFFINITY") == "1" or not hasattr(os, "sched_setaffinity"):
            return None
        try:
            allowed = cls.allowed_cores()
            if len(allowed) < 2 * (n_workers + 1):
                return None          # too few cores to dedicate any
            plan = cls.plan(n_workers, allowed)
            cores = plan[local_index]
            if cores:
                os.sched_setaffinity(0, cores)
                try:        # keep the intra-op pool no larger than the cores it may run on
                    import torch
                    torch.set_num_threads(max(1, min(torch.get_num_threads(), len(cores))))
                except Exception:
                    pass
            return cores
        except Exception:
            return None
