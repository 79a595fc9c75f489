"""Where each teacher parameter's student counterpart lives.

The reference applies the momentum update partition by partition with
``zip(online_params, target_params)`` (`benchmarks/byol/trainer.py:198-212`,
`tspipe/gpu_task.py:403-406`), which silently requires the teacher and the student to be cut at
the same children.  Here the two nets may be cut differently (the forward-only teacher is
cheaper, so a balanced split gives it other boundaries): the i-th teacher parameter in model
order corresponds to the i-th student parameter in model order, wherever that lives.  Per
teacher stage the plan lists contiguous runs of the flat buffers:

``local``   runs whose student source is on the same rank,
``recv``    runs to be read from another stage (its flat student buffer: by point-to-point
            transfer, or through a peer pointer on CUDA),
``send``    runs of this stage's student buffer that other stages need.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

from torch import nn

from .state import ALIGN


def layout_offsets(params: Sequence[nn.Parameter]) -> List[int]:
    offs, off = [], 0
    for p in params:
        offs.append(off)
        off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
    return offs


@dataclass
class EmaPlan:
    local: List[Tuple[int, int, int]] = field(default_factory=list)              # (t_off, s_off, n)
    recv: Dict[int, List[Tuple[int, int, int]]] = field(default_factory=dict)    # src stage -> [(t_off, s_off, n)]
    send: Dict[int, List[Tuple[int, int]]] = field(default_factory=dict)         # dst stage -> [(s_off, n)]

    @property
    def is_local_prefix(self) -> bool:
        return not self.recv and not self.send and len(self.local) <= 1 and \
            (not self.local or (self.local[0][0] == 0 and self.local[0][1] == 0))


def build_ema_plans(partitions_online: Sequence[nn.Module], partitions_target: Sequence[nn.Module]) -> List[EmaPlan]:
    pp = len(partitions_online)
    student: List[Tuple[int, int, int, Tuple[int, ...]]] = []    # (stage, offset, padded_len, shape)
    for j, part in enumerate(partitions_online):
        ps = list(part.parameters())
        for p, off in zip(ps, layout_offsets(ps)):
            student.append((j, off, (p.numel() + ALIGN - 1) // ALIGN * ALIGN, tuple(p.shape)))
    plans = [EmaPlan() for _ in range(max(pp, len(partitions_target)))]
    i = 0
    for jt, part in enumerate(partitions_target):
        ps = list(part.parameters())
        runs: List[List[int]] = []       # [js, t_off, s_off, n]
        for p, t_off in zip(ps, layout_offsets(ps)):
            if i >= len(student):
                raise ValueError("the teacher has more parameters than the student: no momentum counterpart")
            js, s_off, n, shape = student[i]
            if shape != tuple(p.shape):
                raise ValueError(f"teacher parameter {i} has shape {tuple(p.shape)} but its student counterpart "
                                 f"has {shape}: the momentum update needs identical architectures")
            i += 1
            if runs and runs[-1][0] == js and runs[-1][1] + runs[-1][3] == t_off and runs[-1][2] + runs[-1][3] == s_off:
                runs[-1][3] += n
            else:
                runs.append([js, t_off, s_off, n])
        for js, t_off, s_off, n in runs:
            if js == jt:
                plans[jt].local.append((t_off, s_off, n))
            else:
                plans[jt].recv.setdefault(js, []).append((t_off, s_off, n))
                plans[js].send.setdefault(jt, []).append((s_off, n))
    return plans


def split_placement_routes(plans: Sequence[EmaPlan], n_teacher: int, n_student: int
                           ) -> Tuple[List[Dict[int, List[Tuple[int, int, int]]]], List[Dict[int, List[Tuple[int, int]]]]]:
    """The same plan for a job whose teacher stages and student stages live on different ranks: nothing is local.
    Returns ``(sources, dests)``: ``sources[jt][js] = [(t_off, s_off, n)]`` runs teacher stage ``jt`` takes from
    student stage ``js`` (in the order the student packs them), ``dests[js][jt] = [(s_off, n)]`` runs student stage
    ``js`` packs for teacher stage ``jt``."""
    sources: List[Dict[int, List[Tuple[int, int, int]]]] = [dict() for _ in range(n_teacher)]
    dests: List[Dict[int, List[Tuple[int, int]]]] = [dict() for _ in range(n_student)]
    for jt in range(n_teacher):
        plan = plans[jt]
        if plan.local:
            sources[jt].setdefault(jt, []).extend(plan.local)
        for js, runs in plan.recv.items():
            sources[jt].setdefault(js, []).extend(runs)
        for js, runs in sources[jt].items():
            dests[js][jt] = [(s_off, n) for _, s_off, n in runs]
    return sources, dests
