"""Microbatch-aware batch normalisation.

Behaviour of the reference layer (`tspipe/batchnorm.py:17-120`, converter `:122-154`): in
training mode every micro-batch is normalised with its *own* batch statistics, while the
per-channel ``sum`` / ``sum_squares`` / element count are accumulated over ``chunks``
micro-batches and committed to ``running_mean`` / ``running_var`` once per mini-batch
(exponential or cumulative average); evaluation mode uses the running statistics.

The reference pays two extra full reductions over the activation per call (``input.sum`` and
``(input**2).sum``, `:52-53`).  Here the accumulators are fed from the batch statistics the
normalisation computes anyway: ``sum += n*mean`` and ``sum_squares += n*(var + mean^2)`` -
one pass over the activation (on CUDA the sm_100a kernel in :mod:`tspipe_b200.ops.fused`
emits them from its statistics pass; otherwise the statistics come back from the
library call through scratch running buffers with momentum 1).
"""
from __future__ import annotations

from typing import Optional, TypeVar, cast

import torch
import torch.nn.functional as F
from torch import Tensor, nn
from torch.nn.modules.batchnorm import _BatchNorm

TModule = TypeVar("TModule", bound=nn.Module)


class DeferredBatchNorm(_BatchNorm):
    sum: Tensor
    sum_squares: Tensor

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: Optional[float] = 0.1,
                 affine: bool = True, chunks: int = 1) -> None:
        super().__init__(num_features, eps, momentum, affine, track_running_stats=True)
        self.register_buffer("sum", torch.zeros_like(self.running_mean))
        self.register_buffer("sum_squares", torch.zeros_like(self.running_var))
        self.register_buffer("_mb_mean", torch.zeros_like(self.running_mean), persistent=False)
        self.register_buffer("_mb_var", torch.ones_like(self.running_var), persistent=False)
        self.counter = 0
        self.tracked = 0
        self.chunks = chunks
        self.group: Optional["BatchNormGroup"] = None     # set when the partition's statistics are flattened
        self.count: Optional[Tensor] = None
        self._slice = slice(0, num_features)              # this layer's channels inside the group's flat buffers

    def _check_input_dim(self, input: Tensor) -> None:
        if input.dim() < 2:
            raise ValueError(f"expected at least 2D input (got {input.dim()}D input)")

    @torch.no_grad()
    def _track(self, n: int) -> bool:
        """Fold the statistics of the micro-batch just normalised (``_mb_mean`` and the unbiased
        ``_mb_var`` over ``n`` elements per channel) into the mini-batch accumulators."""
        mean = self._mb_mean
        var_b = self._mb_var * ((n - 1) / n) if n > 1 else torch.zeros_like(self._mb_var)
        if self.group is not None:
            from .ops import bn as _bn
            acc = self.group._acc[:, _bn.current_segment_index(), self._slice]     # this view's accumulator set
            acc[0].add_(mean, alpha=n)
            acc[1].add_((var_b + mean * mean), alpha=n)
            acc[2].add_(n)
            return False
        self.sum.add_(mean, alpha=n)
        self.sum_squares.add_((var_b + mean * mean), alpha=n)
        self.counter += n
        self.tracked += 1
        return self.tracked == self.chunks

    @torch.no_grad()
    def _commit(self) -> None:
        self.num_batches_tracked += 1
        m = 1.0 / float(self.num_batches_tracked) if self.momentum is None else self.momentum
        mean = self.sum / self.counter
        var = self.sum_squares / self.counter - mean ** 2
        self.running_mean.mul_(1 - m).add_(mean, alpha=m)
        self.running_var.mul_(1 - m).add_(var, alpha=m)
        self.sum.zero_()
        self.sum_squares.zero_()
        self.counter = 0
        self.tracked = 0

    def forward(self, input: Tensor) -> Tensor:  # type: ignore[override]
        from .ops import bn as _bn
        if input.is_cuda and _bn.applicable(self, input):
            return _bn.bn_act(self, input)
        if self.training and _bn.current_segments() > 1:
            return _bn.bn_act(self, input)          # stacked views: one statistics set per view
        if not self.training:
            return F.batch_norm(input, self.running_mean, self.running_var, self.weight, self.bias,
                                training=False, momentum=0.0, eps=self.eps)
        n = input.numel() // input.size(1)
        out = F.batch_norm(input, self._mb_mean, self._mb_var, self.weight, self.bias,
                           training=True, momentum=1.0, eps=self.eps)
        if self._track(n):
            self._commit()
        return out

    @classmethod
    def convert_deferred_batch_norm(cls, module: TModule, chunks: int = 1) -> TModule:
        """Recursively swap every running-stat ``_BatchNorm`` for a :class:`DeferredBatchNorm`
        sharing its parameters and buffers."""
        if isinstance(module, DeferredBatchNorm):
            module.chunks = chunks
            return cast(TModule, module)
        out: nn.Module = module
        if isinstance(module, _BatchNorm) and module.track_running_stats:
            out = DeferredBatchNorm(module.num_features, module.eps, module.momentum, module.affine, chunks)
            if module.affine:
                out.register_parameter("weight", module.weight)
                out.register_parameter("bias", module.bias)
            out.register_buffer("running_mean", module.running_mean)
            out.register_buffer("running_var", module.running_var)
            out.register_buffer("num_batches_tracked", module.num_batches_tracked)
            out.train(module.training)
        for name, child in module.named_children():
            out.add_module(name, cls.convert_deferred_batch_norm(child, chunks))
        return cast(TModule, out)


class BatchNormGroup:
    """All :class:`DeferredBatchNorm` layers of one partition with their statistics re-homed into flat
    buffers, so that the per-mini-batch commit is a handful of launches for the whole partition instead
    of eight per layer (53 layers in a ResNet-50), and so that nothing on the per-microbatch path depends
    on host-side counters: the kernels accumulate ``sum``, ``sum_squares`` and the per-channel element
    ``count`` on the device.  The owner calls :meth:`step` once per partition forward."""

    def __init__(self, module: nn.Module, chunks: Optional[int] = None):
        self.module = module
        self.layers = [m for m in module.modules() if isinstance(m, DeferredBatchNorm)]
        self.tracked = 0
        self.chunks = chunks if chunks is not None else (self.layers[0].chunks if self.layers else 1)
        if not self.layers:
            return
        dev = self.layers[0].running_mean.device
        total = sum(m.num_features for m in self.layers)
        mk = lambda v=0.0: torch.full((total,), v, dtype=torch.float32, device=dev)
        self.running_mean, self.running_var = mk(), mk(1.0)
        # accumulators as [quantity][set][channel]: set 0 is the one that gets committed; a forward over several
        # stacked views (`step(segments=n)`) lets view g accumulate into set g, `total` elements further on
        self.total, self.max_segments = total, 2
        self._acc = torch.zeros(3, self.max_segments, total, dtype=torch.float32, device=dev)
        self.sum, self.sum_squares, self.count = self._acc[0, 0], self._acc[1, 0], self._acc[2, 0]
        self.momentum = mk()
        self.cma = torch.zeros(total, dtype=torch.bool, device=dev)
        self.nbt = torch.zeros(len(self.layers), dtype=torch.int64, device=dev)
        self.layer_of_channel = torch.empty(total, dtype=torch.int64, device=dev)
        off = 0
        with torch.no_grad():
            for i, m in enumerate(self.layers):
                c = m.num_features
                sl = slice(off, off + c)
                for name, flat in (("running_mean", self.running_mean), ("running_var", self.running_var),
                                   ("sum", self.sum), ("sum_squares", self.sum_squares)):
                    flat[sl].copy_(getattr(m, name))
                    m._buffers[name] = flat[sl]
                self.nbt[i] = m.num_batches_tracked
                m._buffers["num_batches_tracked"] = self.nbt[i]
                m.count = self.count[sl]
                m._slice = sl
                if m.momentum is None:
                    self.cma[sl] = True
                else:
                    self.momentum[sl] = float(m.momentum)
                self.layer_of_channel[sl] = i
                m.group = self
                off += c
        self.any_cma = bool(self.cma.any())

    @torch.no_grad()
    def step(self, segments: int = 1) -> None:
        """One partition forward (one micro- or nano-batch) has been tracked.  ``segments`` > 1: the forward ran
        that many stacked views, each with its own statistics in its own accumulator set; they are tracked one
        after the other, exactly as separate forwards would have been."""
        if not self.layers or not self.module.training:
            return
        for g in range(segments):
            if g > 0:
                self._acc[:, 0] += self._acc[:, g]
                self._acc[:, g].zero_()
            self.tracked += 1
            if self.tracked >= self.chunks:
                self.commit()

    @torch.no_grad()
    def commit(self) -> None:
        self.nbt += 1
        cnt = self.count.clamp_min(1.0)
        mean = self.sum / cnt
        var = self.sum_squares / cnt - mean * mean
        mom = self.momentum
        if self.any_cma:
            mom = torch.where(self.cma, 1.0 / self.nbt[self.layer_of_channel].float(), mom)
        seen = self.count > 0
        self.running_mean.add_(torch.where(seen, (mean - self.running_mean) * mom, torch.zeros_like(mean)))
        self.running_var.add_(torch.where(seen, (var - self.running_var) * mom, torch.zeros_like(var)))
        self.sum.zero_()
        self.sum_squares.zero_()
        self.count.zero_()
        self.tracked = 0
