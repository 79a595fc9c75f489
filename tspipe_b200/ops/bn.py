"""Fused microbatch BatchNorm (+ residual add, + ReLU) over channels-last activations.

Binding of ``csrc/batchnorm.cu``.  :func:`bn_act` is the single entry point used by the models and by
:class:`tspipe_b200.batchnorm.DeferredBatchNorm`; it falls back to the library ops whenever the
fused kernels do not apply (CPU tensors, NCHW layout, channel count not a multiple of 8 ...).
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch.nn.modules.batchnorm import _BatchNorm

from . import fused as _f

_ENABLED = True


def set_enabled(flag: bool) -> None:
    global _ENABLED
    _ENABLED = bool(flag)


_SEGMENTS = 1


class segments:
    """``with segments(2): y = net(torch.cat([view_1, view_2]))`` - every BatchNorm reached through :func:`bn_act`
    normalises each of the ``n`` equal, consecutive groups of rows with that group's own statistics, exactly as
    ``n`` separate forwards would (autograd records the grouping, the backward needs no context)."""

    def __init__(self, n: int):
        self.n, self.prev = int(n), 1

    def __enter__(self):
        global _SEGMENTS
        self.prev, _SEGMENTS = _SEGMENTS, self.n
        return self

    def __exit__(self, *exc):
        global _SEGMENTS
        _SEGMENTS = self.prev
        return False


def current_segments() -> int:
    return _SEGMENTS


_SEG_INDEX = 0      # which view a BatchNorm call belongs to while stacked views are run one after the other


def current_segment_index() -> int:
    return _SEG_INDEX


def _as_rows(x: torch.Tensor) -> Optional[Tuple[int, int]]:
    """(M, C) when ``x`` is laid out as a contiguous [M, C] matrix with channels innermost."""
    if x.dim() == 2 and x.is_contiguous():
        return x.shape[0], x.shape[1]
    if x.dim() == 4:
        n, c, h, w = x.shape
        if h * w == 1:
            return (n, c) if x.is_contiguous() or x.is_contiguous(memory_format=torch.channels_last) else None
        if x.stride() == (h * w * c, 1, w * c, c):
            return n * h * w, c
    return None


def applicable(bn, x: torch.Tensor) -> bool:
    if not (_ENABLED and x.is_cuda and isinstance(bn, _BatchNorm) and bn.affine):
        return False
    if x.dtype not in (torch.float32, torch.bfloat16):
        return False
    mc = _as_rows(x)
    if mc is None:
        return False
    m, c = mc
    if bn.training and m < 2:
        return False
    return c % 8 == 0 and c <= 4096


def _lib():
    L = _f.lib()
    if not hasattr(L, "_bn_ready"):
        for n in ("tsp_bn_stats", "tsp_bn_apply", "tsp_bn_bwd_reduce", "tsp_bn_bwd_apply"):
            getattr(L, n).restype = _c.c_int
        L._bn_ready = True
    return L


def stream_status(reset: bool = False) -> int:
    """0 unless a bounded wait of the streaming statistics kernels ran out on the current device
    (1 = producer, 2 = consumer).  Synchronises the device."""
    L = _lib()
    L.tsp_bn_stream_status.restype = _c.c_int
    return int(L.tsp_bn_stream_status(_c.c_int(1 if reset else 0)))


class _BnAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, relu, eps, fixed, acc_sum, acc_sumsq, acc_count=None, pre_sums=None,
                segs=1, acc_stride=0):
        m, c = _as_rows(x)
        dt = _f._dt(x)
        L = _lib()
        y = torch.empty_like(x)
        if residual is not None:
            if residual.dtype != x.dtype or _as_rows(residual) != (m, c):
                residual = residual.to(x.dtype).contiguous(
                    memory_format=torch.channels_last if x.dim() == 4 else torch.contiguous_format)
        # statistics handed over by the producer of x (a convolution epilogue) replace the statistics pass
        sums = pre_sums if pre_sums is not None else torch.empty(segs * 2 * c, dtype=torch.float32, device=x.device)
        save = torch.empty(segs * 2 * c, dtype=torch.float32, device=x.device)
        wf = weight.detach() if weight.dtype == torch.float32 else weight.detach().float()
        bf = bias.detach() if bias.dtype == torch.float32 else bias.detach().float()
        with _f.on_device(x.device):
            st = _f._stream()
            if fixed is None and pre_sums is None:
                _f._check(L.tsp_bn_stats(_f._ptr(x), _c.c_int64(m), _c.c_int(c), _c.c_int(dt), _f._ptr(sums),
                                         _c.c_int(segs), st), "tsp_bn_stats")
                _f._count(2)
            _f._check(L.tsp_bn_apply(_f._ptr(x), _f._ptr(residual), _f._ptr(y), _f._ptr(sums), _f._ptr(fixed),
                                     _f._ptr(wf), _f._ptr(bf), _f._ptr(save), _f._ptr(acc_sum), _f._ptr(acc_sumsq),
                                     _f._ptr(acc_count), _c.c_int64(acc_stride), _c.c_int64(m), _c.c_int(c),
                                     _c.c_float(eps), _c.c_int(1 if relu else 0), _c.c_int(dt), _c.c_int(segs), st),
                      "tsp_bn_apply")
            _f._count()
        ctx.save_for_backward(x, y if (relu and residual is not None) else None, save, wf, bf)
        ctx.relu, ctx.has_res, ctx.mc, ctx.segs = relu, residual is not None, (m, c), segs
        ctx.wdtype, ctx.bdtype = weight.dtype, bias.dtype
        ctx.fixed = fixed is not None
        ctx.mark_non_differentiable(sums)
        return y, sums

    @staticmethod
    def backward(ctx, dy, _dsums):
        x, y, save, wf, bf = ctx.saved_tensors
        m, c = ctx.mc
        L = _lib()
        dt = _f._dt(x)
        fmt = torch.channels_last if x.dim() == 4 else torch.contiguous_format
        if dy.dtype != x.dtype or _as_rows(dy) != (m, c):
            dy = dy.to(x.dtype).contiguous(memory_format=fmt)
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if (ctx.has_res and ctx.relu) else None
        segs = ctx.segs
        sums = torch.empty(segs * 2 * c, dtype=torch.float32, device=x.device)
        with _f.on_device(x.device):
            st = _f._stream()
            relu = _c.c_int(1 if ctx.relu else 0)
            _f._check(L.tsp_bn_bwd_reduce(_f._ptr(dy), _f._ptr(x), _f._ptr(y), _f._ptr(dres), _f._ptr(save),
                                          _f._ptr(wf), _f._ptr(bf), relu,
                                          _c.c_int64(m), _c.c_int(c), _c.c_int(dt), _f._ptr(sums), _c.c_int(segs), st),
                      "tsp_bn_bwd_reduce")
            if ctx.fixed:
                # evaluation statistics are constants: dx = w * rstd * dy'
                sums_for_dx = torch.zeros_like(sums)
            else:
                sums_for_dx = sums
            src, mask, relu2 = (dres, None, _c.c_int(0)) if dres is not None else (dy, y, relu)
            _f._check(L.tsp_bn_bwd_apply(_f._ptr(src), _f._ptr(x), _f._ptr(mask), _f._ptr(save), _f._ptr(wf),
                                         _f._ptr(bf), relu2, _f._ptr(sums_for_dx), _f._ptr(dx), _c.c_int64(m), _c.c_int(c), _c.c_int(dt),
                                         _c.c_int(segs), st), "tsp_bn_bwd_apply")
            _f._count(3)
        if segs > 1:
            sums = sums.view(segs, 2 * c).sum(0)
        db, dw = sums[:c], sums[c:]
        if ctx.has_res:
            gres = dres if dres is not None else dy
        else:
            gres = None
        return dx, dw.to(ctx.wdtype), db.to(ctx.bdtype), gres, None, None, None, None, None, None, None, None, None


def bn_act(bn, x: torch.Tensor, residual: Optional[torch.Tensor] = None, relu: bool = False,
           sums: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``relu(bn(x) + residual)`` with the statistics semantics of ``bn`` (plain running-stat
    BatchNorm, or :class:`~tspipe_b200.batchnorm.DeferredBatchNorm` whose accumulators are fed by the
    same statistics pass).  ``sums`` = per-channel [sum | sum of squares] of ``x`` when its producer already
    computed them (used in training mode only)."""
    from ..batchnorm import DeferredBatchNorm
    segs = _SEGMENTS if (getattr(bn, "training", False) and isinstance(bn, _BatchNorm)) else 1
    if segs > 1:
        grouped = (isinstance(bn, DeferredBatchNorm) and bn.group is not None and segs <= bn.group.max_segments
                   and x.shape[0] % segs == 0 and applicable(bn, x[: x.shape[0] // segs]) and applicable(bn, x))
        if not grouped:
            # no kernel support for this case: run the groups one after the other
            global _SEG_INDEX
            with segments(1):
                xs = x.chunk(segs)
                rs = residual.chunk(segs) if residual is not None else [None] * segs
                outs = []
                try:
                    for g, (xg, rg) in enumerate(zip(xs, rs)):
                        _SEG_INDEX = g               # the deferred accumulators of view g
                        outs.append(bn_act(bn, xg, rg, relu))
                finally:
                    _SEG_INDEX = 0
                return torch.cat(outs)
        y, _ = _BnAct.apply(x, bn.weight, bn.bias, residual, relu, bn.eps, None, bn.sum, bn.sum_squares, bn.count,
                            sums, segs, bn.group.total)
        return y
    if not applicable(bn, x):
        y = bn(x)
        if residual is not None:
            y = y + residual
        return F.relu(y) if relu else y
    m, c = _as_rows(x)
    if not bn.training or not bn.track_running_stats and False:
        fixed = torch.cat([bn.running_mean.float(), bn.running_var.float()])
        y, _ = _BnAct.apply(x, bn.weight, bn.bias, residual, relu, bn.eps, fixed, None, None)
        return y
    if isinstance(bn, DeferredBatchNorm) and bn.group is not None:
        # the partition's statistics live in flat buffers; the group commits them (one launch set per mini-batch)
        y, _ = _BnAct.apply(x, bn.weight, bn.bias, residual, relu, bn.eps, None, bn.sum, bn.sum_squares, bn.count,
                            sums)
        return y
    if isinstance(bn, DeferredBatchNorm):
        y, _ = _BnAct.apply(x, bn.weight, bn.bias, residual, relu, bn.eps, None, bn.sum, bn.sum_squares, None, sums)
        bn.counter += m
        bn.tracked += 1
        if bn.tracked == bn.chunks:
            bn._commit()
        return y
    y, sums = _BnAct.apply(x, bn.weight, bn.bias, residual, relu, bn.eps, None, None, None, None, sums)
    if bn.track_running_stats and bn.running_mean is not None:
        with torch.no_grad():
            bn.num_batches_tracked += 1
            mom = bn.momentum if bn.momentum is not None else 1.0 / float(bn.num_batches_tracked)
            mean = sums[:c] / m
            var = (sums[c:] / m - mean * mean).clamp_min_(0) * (m / max(m - 1, 1))
            bn.running_mean.mul_(1 - mom).add_(mean.to(bn.running_mean.dtype), alpha=mom)
            bn.running_var.mul_(1 - mom).add_(var.to(bn.running_var.dtype), alpha=mom)
    return y
