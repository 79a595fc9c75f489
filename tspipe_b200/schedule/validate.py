"""Structural checks of a schedule (used by tests and, cheaply, at engine start-up).

The reference has only an ineffective duplicate check (`tspipe/scheduler.py:517-530`,
objects hashed by identity).  These checks are on values.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

from .generator import Op, OpKind, ScheduleSpec, device_program, simulate


class ScheduleError(AssertionError):
    pass


def check_programs(spec: ScheduleSpec, n_batches: int) -> None:
    """Every (net, batch, view, microbatch) exactly once per stage; identical forward and
    backward crossing order on all stages; teacher of batch ``b`` between ``OPT(b-2)`` and
    ``OPT(b-1)`` (one-step-delayed teacher), student of ``b`` after ``OPT(b-1)``."""
    n = spec.n_stages
    fwd_ref: Optional[List[Tuple]] = None
    bwd_ref: Optional[List[Tuple]] = None
    for j in range(n):
        prog = list(device_program(spec, j, 1, n_batches))
        seen = set()
        opt_done = 0
        fwd, bwd = [], []
        for op in prog:
            key = (op.kind, op.batch, op.view, op.ub)
            if key in seen:
                raise ScheduleError(f"stage {j}: {op.short()} scheduled twice")
            seen.add(key)
            if op.kind == OpKind.OPT:
                if op.batch != opt_done + 1:
                    raise ScheduleError(f"stage {j}: OPT out of order at {op.short()}")
                opt_done = op.batch
            elif op.kind == OpKind.T:
                fwd.append(key)
                lo = max(op.batch - 2, min(spec.skip_staleness, op.batch - 1), 0)
                if spec.is_sync_batch(op.batch):
                    lo = op.batch - 1
                if opt_done != lo:
                    raise ScheduleError(f"stage {j}: {op.short()} sees teacher version {opt_done}, expected {lo}")
            elif op.kind == OpKind.O:
                fwd.append(key)
                if opt_done != op.batch - 1:
                    raise ScheduleError(f"stage {j}: {op.short()} sees student version {opt_done}")
            elif op.kind == OpKind.B:
                bwd.append(key)
                if opt_done != op.batch - 1:
                    raise ScheduleError(f"stage {j}: {op.short()} after OPT{opt_done}")
        for b in range(1, n_batches + 1):
            for v in spec.teacher_views:
                for u in range(spec.n_ubatch):
                    if (OpKind.T, b, v, u) not in seen:
                        raise ScheduleError(f"stage {j}: missing T{b}v{v}u{u}")
            for v in spec.student_views:
                for u in range(spec.n_ubatch):
                    if (OpKind.O, b, v, u) not in seen:
                        raise ScheduleError(f"stage {j}: missing O{b}v{v}u{u}")
                for u in range(spec.n_nano):
                    if (OpKind.B, b, v, u) not in seen:
                        raise ScheduleError(f"stage {j}: missing B{b}v{v}u{u}")
            if (OpKind.OPT, b, 0, 0) not in seen:
                raise ScheduleError(f"stage {j}: missing OPT{b}")
        if fwd_ref is None:
            fwd_ref, bwd_ref = fwd, bwd
        elif fwd != fwd_ref or bwd != bwd_ref:
            raise ScheduleError(f"stage {j}: crossing order differs from stage 0")


def steady_state_period(spec: ScheduleSpec, n_batches: int = 8) -> Tuple[int, float]:
    """(clocks between consecutive OPT on stage 0 in steady state, busy fraction there)."""
    table = simulate(spec, n_batches)
    opt_clock: Dict[int, int] = {}
    for c, row in enumerate(table):
        op = row[0]
        if op is not None and op.kind == OpKind.OPT:
            opt_clock[op.batch] = c
    b0, b1 = n_batches - 3, n_batches - 2
    period = opt_clock[b1] - opt_clock[b0]
    lo, hi = opt_clock[b0], opt_clock[b1]
    busy = sum(1 for c in range(lo, hi) for op in table[c] if op is not None)
    return period, busy / (period * spec.n_stages)
