"""Closed-form teacher/student pipeline schedules.

The reference derives its schedule clock by clock with per-device counters
(`tspipe/scheduler.py:51-121` synchronous batch, `:124-165` + `:265-353` warm-up,
`:356-450` steady state, `:553-596` driver) and ships the table to the workers one
RPC per task (`tspipe/tspipe.py:252-363`).  Here the schedule is a pure function
of ``(stage, batch)``: every rank computes *its own column* locally and walks it
without any control-plane traffic.  A unit-time simulator (:func:`simulate`)
turns the per-device programs back into a clock table, which is what the golden
tests compare with the tables produced by the reference generator.

Per-device program (``n`` stages, ``U`` forward microbatches, backward split
``s`` so ``s*U`` backward "nano" batches, two views in self-supervised mode):

* synchronous batch (GPipe emulation, or the first ``num_skip_initial_staleness``
  batches):  ``T(b) .. O(b) .. [LOSS] B(b) .. OPT(b)``
* pipelined batch ``b``:  ``O(b) ..  T(b+1)[:k_j]  [LOSS]  B(b) ..  T(b+1)[k_j:]  OPT(b)``
  where ``k_j`` teacher forwards of the *next* batch fill the bubble before the
  backward wave reaches stage ``j`` and the rest fill the tail after it left.

Because every ``T(b+1)`` on a device sits between ``OPT(b-1)`` and ``OPT(b)``,
the teacher it sees is exactly "version ``b-1``" - the one-step-delayed momentum
teacher (`tspipe/gpu_task.py:58-66`) - by construction, with no parameter
versioning needed on the device.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum
from typing import Dict, Iterator, List, Optional, Sequence, Tuple


class OpKind(IntEnum):
    T = 0      # teacher forward of one microbatch
    O = 1      # student ("online") forward of one microbatch
    B = 2      # student backward of one nano-batch
    LOSS = 3   # loss + output gradients (last stage only)
    OPT = 4    # optimizer step (+ momentum-teacher update)


@dataclass(frozen=True)
class Op:
    kind: OpKind
    batch: int          # 1-based batch id, as in the reference (`tspipe/batch_ops.py:258`)
    view: int = 0
    ub: int = 0         # forward microbatch id, or backward nano-batch id for B
    stage: int = 0

    def short(self) -> str:
        if self.kind == OpKind.OPT:
            return f"OPT{self.batch}"
        if self.kind == OpKind.LOSS:
            return f"L{self.batch}"
        return f"{self.kind.name}{self.batch}v{self.view}u{self.ub}"


@dataclass(frozen=True)
class ScheduleSpec:
    """Everything the schedule depends on.

    ``kd`` selects the supervised / frozen-or-momentum KD filter: the teacher only
    sees view 1 and the student only view 0 (`tspipe/tspipe.py:310-320`).
    ``gpipe`` reproduces ``gpipe_emulation.enabled``: every batch synchronous and
    the backward uses the same microbatch count as the forward
    (`tspipe/tspipe.py:106-111`).
    """
    n_stages: int
    n_ubatch: Optional[int] = None       # default: n_stages - 1 (reference), min 1
    bwd_split: int = 2                   # nano-batches per forward microbatch
    kd: bool = False
    skip_staleness: int = 0
    gpipe: bool = False

    def __post_init__(self):
        if self.n_stages < 1:
            raise ValueError("n_stages must be >= 1")
        u = self.n_ubatch
        if u is None:
            u = max(self.n_stages - 1, 1)
            object.__setattr__(self, "n_ubatch", u)
        if u < 1 or self.bwd_split < 1:
            raise ValueError("n_ubatch and bwd_split must be >= 1")
        if self.gpipe:
            object.__setattr__(self, "bwd_split", 1)

    # -- item lists -------------------------------------------------------------------------
    @property
    def teacher_views(self) -> Tuple[int, ...]:
        return (1,) if self.kd else (0, 1)

    @property
    def student_views(self) -> Tuple[int, ...]:
        return (0,) if self.kd else (0, 1)

    @property
    def n_nano(self) -> int:
        return self.n_ubatch * self.bwd_split

    def is_sync_batch(self, batch: int) -> bool:
        return self.gpipe or batch <= self.skip_staleness

    def teacher_items(self, batch: int, stage: int) -> List[Op]:
        return [Op(OpKind.T, batch, v, u, stage) for v in self.teacher_views for u in range(self.n_ubatch)]

    def student_items(self, batch: int, stage: int) -> List[Op]:
        return [Op(OpKind.O, batch, v, u, stage) for v in self.student_views for u in range(self.n_ubatch)]

    def backward_items(self, batch: int, stage: int) -> List[Op]:
        return [Op(OpKind.B, batch, v, u, stage)
                for v in reversed(self.student_views) for u in reversed(range(self.n_nano))]

    def teacher_head(self, stage: int) -> int:
        """Number of next-batch teacher forwards placed *before* the backward wave.

        After stage ``j`` finishes its last student forward the wave needs ``n-1-j``
        forward hops down (one slot each) and ``n-1-j`` backward hops back, a backward
        item costing ``2 / bwd_split`` forward slots: with the reference's split of 2
        that is ``2(n-1-j)`` free slots, with unsplit backwards ``3(n-1-j)``.  In
        the SSL table the slots are consecutive teacher items; under the KD filter
        the dropped view-0 items come first, so only the view-1 part survives.
        """
        hops = self.n_stages - 1 - stage
        free = hops + (2 * hops + self.bwd_split - 1) // self.bwd_split
        full = 2 * self.n_ubatch
        head_ssl = min(free, full)
        if not self.kd:
            return head_ssl
        return max(0, head_ssl - self.n_ubatch)   # items [U, 2U) of the SSL order are view 1


def batch_block(spec: ScheduleSpec, stage: int, batch: int, last_batch: Optional[int] = None,
                fill: Optional[bool] = None) -> List[Op]:
    """Ordered ops of stage ``stage`` attributed to ``batch``.

    ``last_batch`` (set once the feeder has stopped) removes the look-ahead teacher
    forwards of a batch that will never be fed.  ``fill`` marks a batch whose teacher
    forwards were not produced as look-ahead of the previous block (the first pipelined
    batch, or the first batch after the pipeline was flushed); default: the first
    pipelined batch only.
    """
    last = stage == spec.n_stages - 1
    ops: List[Op] = []
    loss = [Op(OpKind.LOSS, batch, 0, 0, stage)] if last else []
    opt = [Op(OpKind.OPT, batch, 0, 0, stage)]
    if spec.is_sync_batch(batch):
        return (spec.teacher_items(batch, stage) + spec.student_items(batch, stage) + loss
                + spec.backward_items(batch, stage) + opt)
    if fill is None:
        fill = batch == spec.skip_staleness + 1
    if fill:
        ops += spec.teacher_items(batch, stage)        # pipeline fill: nothing earlier produced T(b)
    ops += spec.student_items(batch, stage)
    nxt = spec.teacher_items(batch + 1, stage) if (last_batch is None or batch + 1 <= last_batch) else []
    k = spec.teacher_head(stage)
    ops += nxt[:k] + loss + spec.backward_items(batch, stage) + nxt[k:] + opt
    return ops


def device_program(spec: ScheduleSpec, stage: int, first_batch: int = 1,
                   last_batch: Optional[int] = None) -> Iterator[Op]:
    """Infinite (or bounded by ``last_batch``) op stream of one stage."""
    b = first_batch
    while last_batch is None or b <= last_batch:
        yield from batch_block(spec, stage, b, last_batch)
        b += 1


def forward_order(spec: ScheduleSpec, first_batch: int, last_batch: int) -> List[Op]:
    """Order in which forward activations cross every stage boundary (stage field = 0).

    The subsequence of T/O items is identical on all stages, which is what lets a
    receiver post its NCCL receives ahead of time in the sender's order.
    """
    return [op for op in device_program(spec, 0, first_batch, last_batch) if op.kind in (OpKind.T, OpKind.O)]


def backward_order(spec: ScheduleSpec, first_batch: int, last_batch: int) -> List[Op]:
    return [op for op in device_program(spec, 0, first_batch, last_batch) if op.kind == OpKind.B]


# ---------------------------------------------------------------------------------------------
# unit-time simulation -> clock table
# ---------------------------------------------------------------------------------------------
def simulate(spec: ScheduleSpec, n_batches: int, lockstep_opt: bool = False) -> List[List[Optional[Op]]]:
    """Greedy unit-time execution of the per-device programs.

    Every op takes one clock; a forward item at stage ``j`` may run one clock after
    stage ``j-1`` ran it, a backward item one clock after stage ``j+1`` ran it (LOSS
    is folded into the first backward of the last stage, as in the reference table).
    Returns ``table[clock][stage]``.
    """
    n = spec.n_stages
    progs = [[op for op in device_program(spec, j, 1, n_batches) if op.kind != OpKind.LOSS] for j in range(n)]
    pos = [0] * n
    done: Dict[Tuple, int] = {}
    table: List[List[Optional[Op]]] = []
    clock = 0
    total = sum(len(p) for p in progs)
    executed = 0
    while executed < total:
        row: List[Optional[Op]] = [None] * n
        for j in range(n):
            if pos[j] >= len(progs[j]):
                continue
            op = progs[j][pos[j]]
            ready = True
            if op.kind in (OpKind.T, OpKind.O) and j > 0:
                t = done.get((op.kind, op.batch, op.view, op.ub, j - 1))
                ready = t is not None and t < clock
            elif op.kind == OpKind.B and j < n - 1:
                t = done.get((op.kind, op.batch, op.view, op.ub, j + 1))
                ready = t is not None and t < clock
            if ready:
                row[j] = op
        for j, op in enumerate(row):
            if op is not None:
                done[(op.kind, op.batch, op.view, op.ub, j)] = clock
                pos[j] += 1
                executed += 1
        if all(r is None for r in row):
            raise RuntimeError(f"schedule deadlock at clock {clock}: {[p[i] if i < len(p) else None for p, i in zip(progs, pos)]}")
        table.append(row)
        clock += 1
    return table


def format_table(table: Sequence[Sequence[Optional[Op]]]) -> str:
    lines = []
    for c, row in enumerate(table):
        lines.append(f"{c:4d} | " + " | ".join((op.short() if op else ".").ljust(9) for op in row))
    return "\n".join(lines)
