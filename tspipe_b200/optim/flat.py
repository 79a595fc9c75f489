"""Optimizers that step a whole partition's flat parameter buffer in one or two launches.

``LARS`` follows `benchmarks/byol/main.py:13-46` (no trust-ratio scaling or weight decay for
parameters with ``ndim <= 1``), ``AdamW`` and ``SGD`` follow ``torch.optim`` (what
`benchmarks/distilbert/distiller.py:150` and `benchmarks/soft_target/train_kd.py:209-213` use).
They are ordinary ``torch.optim.Optimizer`` subclasses - usable on their own, per tensor - and
gain the fused path when the engine calls :meth:`bind_flat` with the partition's
:class:`~tspipe_b200.runtime.state.FlatParams`: state lives in flat buffers too, per-tensor
hyper-parameters go into a small table, and on CUDA the sm_100a kernels of
``csrc/flat_optim.cu`` do the work.  With ``fuse_ema`` the momentum-teacher update of the
corresponding local teacher buffer rides in the same launch.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch
from torch.optim import Optimizer


class _FlatMixin:
    flat = None
    use_kernel = False
    handles_dp = False

    def bind_flat(self, flat, use_kernel: bool) -> None:
        self.flat, self.use_kernel = flat, bool(use_kernel)
        self._seg_group: List[Dict[str, Any]] = []
        by_id = {}
        for g in self.param_groups:
            for p in g["params"]:
                by_id[id(p)] = g
        for p in flat.params:
            if id(p) not in by_id:
                raise ValueError("a partition parameter is missing from the optimizer's param groups")
            self._seg_group.append(by_id[id(p)])
        self._flat_state: Dict[str, torch.Tensor] = {}
        self._steps = 0
        self.teacher_flat: Optional[torch.Tensor] = None     # set by the engine to fuse the EMA
        self.ema_momentum = 0.0
        if self.use_kernel:
            from ..ops import fused
            self._chunks = fused.build_chunks(flat.offsets, flat.numels, flat.device)
            self._norms = torch.zeros(2 * max(len(flat.params), 1), dtype=torch.float32, device=flat.device)
        self._hp_cache = None

    def enable_dp(self, group, peer_grads, peer_params, self_index: int) -> None:
        """Data-parallel mode over peer-mapped buffers: this rank owns ``1/R`` of the flat range; the step
        sums that range of every replica's gradients with peer loads, updates it, and stores the new
        parameters into every replica's buffer (``csrc/peer.cu``).  ``peer_grads`` / ``peer_params`` hold one
        flat tensor per replica (this rank's own at ``self_index``)."""
        from ..comm.peer import pointer_table
        from ..ops import fused
        assert self.flat is not None and self.use_kernel
        r = len(peer_grads)
        assert self.flat.total % r == 0
        shard = self.flat.total // r
        self._dp = dict(group=group, r=r, idx=self_index, grads=pointer_table(peer_grads),
                        params=pointer_table(peer_params), keep=(list(peer_grads), list(peer_params)),
                        chunks=fused.build_chunks(self.flat.offsets, self.flat.numels, self.flat.device,
                                                  self_index * shard, (self_index + 1) * shard),
                        token=torch.zeros(1, device=self.flat.device), phase=0, reduced=False, signals=None)
        self.handles_dp = True

    def enable_signals(self, pad, norm_tables=None) -> None:
        """Order the data-parallel kernels with device-side signals (:class:`tspipe_b200.comm.signals.SignalPad`)
        instead of tiny NCCL collectives; ``norm_tables`` = every replica's ``[R][2 * n_tensors]`` table through
        which LARS exchanges its partial norms with peer stores."""
        from ..comm.peer import pointer_table
        d = self._dp
        d["signals"] = pad
        if norm_tables is not None:
            d["norm_tables"] = pointer_table(norm_tables)
            d["norm_keep"] = list(norm_tables)
            d["norm_table"] = norm_tables[d["idx"]]

    def _dp_barrier(self) -> None:
        """All replicas have reached this point of their streams (and what they enqueued before it is visible)."""
        d = self._dp
        if d["signals"] is not None:
            d["phase"] += 1
            d["signals"].arrive(d["phase"])
            d["signals"].wait(d["phase"])
            return
        import torch.distributed as dist
        dist.all_reduce(d["token"], group=d["group"])

    def dp_reduce(self, grad_scale: float = 1.0) -> None:
        """First half of the data-parallel step, callable as soon as this replica's backward is complete (and on
        another stream than the one that goes on computing): wait for every replica's backward, sum this rank's
        range of all gradient buffers, and for LARS exchange the partial norms.  :meth:`step` skips this half when
        it has already run for the step."""
        raise NotImplementedError

    def _buf(self, name: str) -> torch.Tensor:
        if name not in self._flat_state:
            self._flat_state[name] = torch.zeros_like(self.flat.data)
        return self._flat_state[name]

    def _views(self, flat_tensor: torch.Tensor, i: int) -> torch.Tensor:
        return self.flat._view(flat_tensor, i, self.flat.params[i].data)

    def _hp_table(self, rows: List[List[float]]) -> torch.Tensor:
        key = tuple(tuple(r) for r in rows)
        if self._hp_cache is None or self._hp_cache[0] != key:
            self._hp_cache = (key, torch.tensor(rows, dtype=torch.float32, device=self.flat.device))
        return self._hp_cache[1]

    def flat_state_dict(self) -> Dict[str, Any]:
        return {"flat": {k: v.detach().cpu() for k, v in self._flat_state.items()}, "steps": self._steps}

    def shard_range(self) -> Optional[tuple]:
        """``(lo, hi)``: the range of the flat buffers this replica updates in data-parallel mode (the state
        outside it is never touched here and stays zero); None when the whole state is local."""
        if not self.handles_dp or self.flat is None:
            return None
        r, idx = self._dp["r"], self._dp["idx"]
        shard = self.flat.total // r
        return idx * shard, (idx + 1) * shard

    def flat_shard_state(self) -> Optional[Dict[str, Any]]:
        """This replica's range of every flat state buffer (for per-replica checkpoint files)."""
        rng = self.shard_range()
        if rng is None:
            return None
        lo, hi = rng
        return {"lo": lo, "hi": hi, "total": self.flat.total, "steps": self._steps,
                "flat": {k: v[lo:hi].detach().cpu().clone() for k, v in self._flat_state.items()}}

    def load_flat_shards(self, pieces: List[Dict[str, Any]]) -> None:
        """Reassemble the flat state from per-replica ranges (any number of them, any replica count now)."""
        if self.flat is None:
            return
        for piece in pieces:
            if piece.get("total") != self.flat.total:
                raise ValueError("optimizer shard was written for a different partition layout")
            for k, v in piece["flat"].items():
                self._buf(k)[piece["lo"]: piece["hi"]].copy_(v)
            self._steps = max(self._steps, int(piece["steps"]))

    def state_dict(self):  # type: ignore[override]
        sd = super().state_dict()
        if self.flat is not None:
            sd["tspipe_flat"] = self.flat_state_dict()
        return sd

    def load_state_dict(self, sd):  # type: ignore[override]
        extra = None
        if isinstance(sd, dict) and "tspipe_flat" in sd:
            sd = dict(sd)                      # the caller's dict stays as it was
            extra = sd.pop("tspipe_flat")
        super().load_state_dict(sd)
        if extra is not None and self.flat is not None:
            for k, v in extra["flat"].items():
                self._buf(k).copy_(v)
            self._steps = extra["steps"]


class LARS(_FlatMixin, Optimizer):
    def __init__(self, params, lr=0, weight_decay=0, momentum=0.9, trust_coefficient=0.001):
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, momentum=momentum,
                                      trust_coefficient=trust_coefficient))

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        if self.flat is None:
            return self._step_per_tensor()
        flat = self.flat
        self._steps += 1
        mu = self._buf("mu")
        if self.use_kernel:
            from ..ops import fused
            rows = [[g["lr"], g["weight_decay"], g["momentum"], g["trust_coefficient"], 1.0 if p.ndim > 1 else 0.0]
                    for p, g in zip(flat.params, self._seg_group)]
            if self.handles_dp:
                d = self._dp
                hp = self._hp_table(rows)
                if not d["reduced"]:
                    self.dp_reduce(grad_scale)
                d["reduced"] = False
                if d["signals"] is not None and "norm_table" in d:
                    d["signals"].wait(d["phase"])       # every replica's norms are here and all gradient reads done
                    fused.sum_norms_(d["norm_table"], d["r"], self._norms)
                fused.dp_lars_apply_(d["params"], d["r"], d["idx"], flat.grad, mu, d["chunks"], hp, self._norms)
                self._dp_barrier()                      # every replica's parameters are complete
                return
            fused.lars_step_(flat.data, flat.grad, mu, self._chunks, self._hp_table(rows), self._norms, grad_scale,
                             self.teacher_flat, self.ema_momentum)
            return
        for i, (p, g) in enumerate(zip(flat.params, self._seg_group)):
            self._lars_one(p, self._views(flat.grad, i) * grad_scale, self._views(mu, i), g)
        if self.teacher_flat is not None:
            n = self.teacher_flat.numel()
            self.teacher_flat.lerp_(flat.data[:n], 1.0 - self.ema_momentum)

    @torch.no_grad()
    def dp_reduce(self, grad_scale: float = 1.0) -> None:
        import torch.distributed as dist
        from ..ops import fused
        flat, d = self.flat, self._dp
        rows = [[g["lr"], g["weight_decay"], g["momentum"], g["trust_coefficient"], 1.0 if p.ndim > 1 else 0.0]
                for p, g in zip(flat.params, self._seg_group)]
        hp = self._hp_table(rows)
        self._dp_barrier()                              # every replica's backward is complete
        fused.dp_reduce_norms_(d["grads"], d["r"], grad_scale / d["r"], flat.grad, flat.data, d["chunks"], hp,
                               self._norms)
        if d["signals"] is not None and "norm_table" in d:
            # partial norms to every replica's table, then the signal that they (and this rank's reads) are done
            fused.publish_norms_(d["norm_tables"], d["r"], d["idx"], self._norms)
            d["phase"] += 1
            d["signals"].arrive(d["phase"])
        else:
            dist.all_reduce(self._norms, group=d["group"])     # whole-tensor norms; also: all gradient reads done
        d["reduced"] = True

    @staticmethod
    def _lars_one(p, dp, mu, g):
        if p.ndim > 1:
            dp = dp.add(p, alpha=g["weight_decay"])
            pn, un = torch.norm(p), torch.norm(dp)
            one = torch.ones_like(pn)
            q = torch.where(pn > 0., torch.where(un > 0, g["trust_coefficient"] * pn / un, one), one)
            dp = dp.mul(q)
        mu.mul_(g["momentum"]).add_(dp)
        p.add_(mu, alpha=-g["lr"])

    def _step_per_tensor(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "mu" not in st:
                    st["mu"] = torch.zeros_like(p)
                self._lars_one(p, p.grad, st["mu"], g)


class AdamW(_FlatMixin, Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        if self.flat is None:
            return self._step_per_tensor()
        flat = self.flat
        self._steps += 1
        t = self._steps
        m, v = self._buf("exp_avg"), self._buf("exp_avg_sq")
        if self.use_kernel:
            from ..ops import fused
            rows = [[g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"],
                     1.0 - g["betas"][0] ** t, 1.0 - g["betas"][1] ** t] for g in self._seg_group]
            if self.handles_dp:
                d = self._dp
                if not d["reduced"]:
                    self.dp_reduce(grad_scale)
                d["reduced"] = False
                if d["signals"] is not None:
                    d["signals"].wait(d["phase"])       # every replica's backward is complete
                fused.dp_adamw_step_(d["grads"], d["params"], d["r"], d["idx"], grad_scale / d["r"], m, v, d["chunks"],
                                     self._hp_table(rows))
                self._dp_barrier()
                return
            fused.adamw_step_(flat.data, flat.grad, m, v, self._chunks, self._hp_table(rows), grad_scale,
                              self.teacher_flat, self.ema_momentum)
            return
        for i, (p, g) in enumerate(zip(flat.params, self._seg_group)):
            self._adamw_one(p, self._views(flat.grad, i) * grad_scale, self._views(m, i), self._views(v, i), g, t)
        if self.teacher_flat is not None:
            n = self.teacher_flat.numel()
            self.teacher_flat.lerp_(flat.data[:n], 1.0 - self.ema_momentum)

    @torch.no_grad()
    def dp_reduce(self, grad_scale: float = 1.0) -> None:
        """AdamW reduces, updates and stores in one kernel, so its early half only announces that this replica's
        gradients are complete (with signals) or waits for all of them (collectives)."""
        d = self._dp
        if d["signals"] is not None:
            d["phase"] += 1
            d["signals"].arrive(d["phase"])
        else:
            self._dp_barrier()
        d["reduced"] = True

    @staticmethod
    def _adamw_one(p, grad, m, v, g, t):
        b1, b2 = g["betas"]
        p.mul_(1.0 - g["lr"] * g["weight_decay"])
        m.mul_(b1).add_(grad, alpha=1 - b1)
        v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
        denom = (v.sqrt() / math.sqrt(bc2)).add_(g["eps"])
        p.addcdiv_(m, denom, value=-g["lr"] / bc1)

    def _step_per_tensor(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"], st["exp_avg"], st["exp_avg_sq"] = 0, torch.zeros_like(p), torch.zeros_like(p)
                st["step"] += 1
                self._adamw_one(p, p.grad, st["exp_avg"], st["exp_avg_sq"], g, st["step"])


class SGD(_FlatMixin, Optimizer):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False):
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov))

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        if self.flat is None:
            return self._step_per_tensor()
        flat = self.flat
        self._steps += 1
        first = self._steps == 1
        buf = self._buf("momentum_buffer")
        if self.use_kernel:
            from ..ops import fused
            rows = [[g["lr"], g["momentum"], g["dampening"], g["weight_decay"], 1.0 if g["nesterov"] else 0.0,
                     1.0 if first else 0.0] for g in self._seg_group]
            fused.sgd_step_(flat.data, flat.grad, buf, self._chunks, self._hp_table(rows), grad_scale,
                            self.teacher_flat, self.ema_momentum)
            return
        for i, (p, g) in enumerate(zip(flat.params, self._seg_group)):
            self._sgd_one(p, self._views(flat.grad, i) * grad_scale, self._views(buf, i), g, first)
        if self.teacher_flat is not None:
            n = self.teacher_flat.numel()
            self.teacher_flat.lerp_(flat.data[:n], 1.0 - self.ema_momentum)

    @staticmethod
    def _sgd_one(p, d, buf, g, first):
        if g["weight_decay"] != 0:
            d = d.add(p, alpha=g["weight_decay"])
        if g["momentum"] != 0:
            if first:
                buf.copy_(d)
            else:
                buf.mul_(g["momentum"]).add_(d, alpha=1 - g["dampening"])
            d = d.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
        p.add_(d, alpha=-g["lr"])

    def _step_per_tensor(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                first = "momentum_buffer" not in st
                if first:
                    st["momentum_buffer"] = torch.zeros_like(p)
                self._sgd_one(p, p.grad, st["momentum_buffer"], g, first)
