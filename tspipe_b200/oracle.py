"""Single-process numerical oracle: what the pipelined runtime must compute.

Semantics (reference: `tspipe/gpu_task.py:58-66` version rule, `:89-226` full-batch loss,
`:229-285` per-nano-batch backward with summed parameter gradients, `:322-417` step + EMA):

* student of batch ``b`` runs with the parameters after ``OPT(b-1)``;
* teacher of batch ``b`` runs with the teacher after ``OPT(max(b-2, s))`` (``b-1`` during the
  ``s`` synchronous warm-up batches and in GPipe emulation): the one-step-delayed teacher;
* forward runs microbatch by microbatch (nano-batch by nano-batch for the student), so
  BatchNorm sees microbatch statistics; the loss is evaluated once on the gathered full batch;
* ``teacher_k = update_fn(momentum, student_k, teacher_{k-1})``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch
from torch import nn
from torch.func import functional_call


def _chunks(x: torch.Tensor, n: int) -> List[torch.Tensor]:
    return list(x.chunk(n))


class DelayedTeacherOracle:
    def __init__(self, online: nn.Module, target: nn.Module, optimizer: torch.optim.Optimizer, loss_fn: Callable,
                 target_update_fn: Optional[Callable], momentum: float, kd: bool, n_ubatch: int, bwd_split: int = 2,
                 skip_staleness: int = 0, gpipe: bool = False, extra_args: Any = None, args: Any = None,
                 gradient_accumulation: int = 1):
        self.online, self.target, self.opt, self.loss_fn = online, target, optimizer, loss_fn
        self.update_fn, self.momentum, self.kd = target_update_fn, momentum, kd
        self.U, self.S = n_ubatch, (1 if gpipe else bwd_split)
        self.skip, self.gpipe = skip_staleness, gpipe
        self.extra_args, self.args = extra_args, args
        self.ga, self.ga_count = gradient_accumulation, 0
        self.b = 0
        self.teacher_versions: Dict[int, Dict[str, torch.Tensor]] = {0: self._snap()}
        for p in self.target.parameters():
            p.requires_grad_(False)

    def _snap(self) -> Dict[str, torch.Tensor]:
        return {k: v.detach().clone() for k, v in self.target.named_parameters()}

    def _teacher_version(self, b: int) -> int:
        if self.gpipe or b <= self.skip + 1:
            return max(b - 1, 0)
        return max(b - 2, self.skip)

    def _teacher_forward(self, b: int, x: torch.Tensor) -> torch.Tensor:
        params = self.teacher_versions[self._teacher_version(b)]
        outs = []
        with torch.no_grad():
            for c in _chunks(x, self.U):
                outs.append(functional_call(self.target, params, (c,)))
        return torch.cat(outs)

    def _student_forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.cat([self.online(c) for u in _chunks(x, self.U) for c in _chunks(u, self.S)])

    def step(self, view_1: torch.Tensor, view_2: torch.Tensor, labels: Any = None, force_step: bool = False,
             epoch: int = 0) -> float:
        self.b += 1
        b = self.b
        if self.kd:
            t = self._teacher_forward(b, view_2)
            o = self._student_forward(view_1)
            loss = self.loss_fn(o, t, labels, self.args, self.extra_args, epoch)
        else:
            t1 = self._teacher_forward(b, view_1)
            t2 = self._teacher_forward(b, view_2)
            o1 = self._student_forward(view_1)
            o2 = self._student_forward(view_2)
            loss = self.loss_fn(o1, o2, t1, t2, self.args, self.extra_args)
        loss.backward()
        if (self.ga_count + 1) % self.ga != 0 and not force_step:
            self.ga_count += 1
        else:
            if self.ga > 1:
                for p in self.online.parameters():
                    if p.grad is not None:
                        p.grad /= (self.ga_count + 1)
                self.ga_count = 0
            self.opt.step()
            self.opt.zero_grad()
        prev = self.teacher_versions[b - 1]
        if self.update_fn is None:
            self.teacher_versions[b] = prev
        else:
            names = [k for k, _ in self.target.named_parameters()]
            online_params = [p.detach() for p in self.online.parameters()]
            new = self.update_fn(self.momentum, online_params, [prev[k] for k in names])
            self.teacher_versions[b] = {k: v.detach().clone() for k, v in zip(names, new)}
        self.teacher_versions.pop(b - 3, None)
        return float(loss.detach())

    def final_teacher(self) -> Dict[str, torch.Tensor]:
        return self.teacher_versions[self.b]
