"""A pipeline stage's forward and backward as CUDA graphs.

A ResNet-50 stage is a few hundred small launches per microbatch; at 128 samples per GPU the Python side of those
launches (autograd bookkeeping, allocation, argument marshalling) costs about as much time as the kernels take to
run, and with more microbatches per step the host becomes the bound.  Here the launch sequence of a stage is
recorded once per (microbatch slot, input geometry) and replayed with one call:

* the FORWARD of the student stage is captured with autograd recording, from static copies of the stage's input
  tensors; directly afterwards the BACKWARD is captured into a second graph of the same memory pool with
  ``torch.autograd.grad`` from static output-gradient buffers, and its parameter gradients are added to the
  parameters' ``.grad`` views (the partition's flat gradient buffer) inside the graph;
* a replay of the forward copies the microbatch into the static inputs, launches the graph and hands out copies of
  the static outputs; a replay of the backward copies the received output gradients in, launches, and hands out
  copies of the input gradients.  The activations saved between the two live in the graph's pool, at the same
  addresses every step;
* one pair of graphs (and one pool) per microbatch slot, because the forwards of all microbatches of a batch run
  before their backwards; a slot that is asked to run a second forward before its backward falls back to eager.

Weights are cast to bf16 inside the graphs (the per-step weight caches are bypassed while capturing,
``ops.fused.capturing``), BatchNorm statistics accumulate in device buffers; nothing inside a stage may depend on
host state.  Stages with active dropout, skip connections, BatchNorm layers outside a
:class:`~tspipe_b200.batchnorm.BatchNormGroup`, or gradients outside the flat buffer are not captured.

Capture runs on a private stream that is ordered after the caller's stream, in thread-local capture mode and
without a device-wide synchronisation: other streams of a pipelined rank may hold a (bounded) device-side wait for
a message that only arrives after this rank has made progress.

The reference runs every operation eagerly and synchronises the device around each task
(`tspipe/gpu_task.py:180,204`).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn

from ..ops import fused as _f
from ..utils import pytree as pt

WARMUP_CALLS = 2          # eager calls per slot before capture (library autotuning, lazy initialisation)


def capture(graph: "torch.cuda.CUDAGraph", stream: "torch.cuda.Stream", pool, body):
    """Record ``body()`` into ``graph`` on ``stream`` (ordered after the current stream).  Returns ``body``'s value."""
    cur = torch.cuda.current_stream()
    stream.wait_stream(cur)
    with torch.cuda.stream(stream):
        graph.capture_begin(pool=pool, capture_error_mode="thread_local")
        try:
            with _f.capturing():
                out = body()
        except BaseException:
            try:
                graph.capture_end()
            except Exception:
                pass
            raise
        graph.capture_end()
    cur.wait_stream(stream)
    return out


def stage_is_capturable(module: nn.Module) -> bool:
    from torch.nn.modules.batchnorm import _BatchNorm
    from ..batchnorm import DeferredBatchNorm
    for m in module.modules():
        if isinstance(m, nn.Dropout) and m.p > 0 and m.training:
            return False
        if isinstance(m, _BatchNorm) and m.training:
            if not (isinstance(m, DeferredBatchNorm) and m.group is not None):
                return False
        if type(m).__name__ in ("Skippable", "Portal") or hasattr(m, "stashable_names"):
            return False
    return True


class _Slot:
    __slots__ = ("calls", "fwd", "bwd", "pool", "static_in", "tpos", "static_out", "out_flags", "static_gout",
                 "static_gin", "launches_f", "launches_b", "busy", "failed")

    def __init__(self):
        self.calls, self.fwd, self.bwd, self.busy, self.failed = 0, None, None, False, False


class StudentStageGraphs:
    """Graph pairs of one student partition, keyed by (slot, input geometry, stacked views)."""

    def __init__(self, module: nn.Module, flat, autocast: bool, device: torch.device):
        self.module, self.autocast, self.device = module, bool(autocast), device
        self.params = [p for p in flat.params if p.requires_grad]
        esz = flat.grad.element_size() if flat.grad is not None else 4
        self.enabled = flat.grad is not None and all(
            p.grad is not None and p.grad.data_ptr() == flat.grad.data_ptr() + esz * off
            for p, off in zip(flat.params, flat.offsets) if p.requires_grad)
        self.stream = torch.cuda.Stream(device)
        self.slots: Dict[Any, _Slot] = {}

    # -- forward -------------------------------------------------------------------------------------
    def forward(self, slot_id: Any, x: Any, segs: int) -> Tuple[Any, Optional[_Slot]]:
        """``(y, slot)`` from the slot's graph, or ``(None, None)`` when the caller has to run the stage eagerly
        (warm-up calls, unsupported input, a slot whose backward has not run yet)."""
        if not self.enabled or not self.module.training:
            return None, None
        leaves, tree, wrapped = pt.flatten(x)
        tpos = [i for i, l in enumerate(leaves) if isinstance(l, torch.Tensor)]
        if not tpos or any(not leaves[i].is_cuda for i in tpos):
            return None, None
        key = (slot_id, segs, str(tree), wrapped,
               tuple((tuple(leaves[i].shape), leaves[i].dtype, leaves[i].stride(), leaves[i].requires_grad)
                     for i in tpos),
               tuple(repr(l) for i, l in enumerate(leaves) if i not in tpos))
        slot = self.slots.get(key)
        if slot is None:
            slot = self.slots[key] = _Slot()
            if not stage_is_capturable(self.module):
                slot.failed = True
        if slot.failed or slot.busy:
            return None, None
        if slot.calls < WARMUP_CALLS:
            slot.calls += 1
            return None, None
        if slot.fwd is None:
            try:
                self._capture(slot, leaves, tpos, tree, wrapped, segs)
            except Exception as e:  # noqa: BLE001 - a stage that cannot be recorded keeps running eagerly
                slot.failed = True
                slot.fwd = slot.bwd = None
                from ..logger import Log
                Log.w(f"stage not captured into CUDA graphs ({type(e).__name__}: {e}); it stays on the eager path")
                return None, None
        with torch.no_grad():
            for i in tpos:
                slot.static_in[i].copy_(leaves[i])
        slot.fwd.replay()
        _f._count(slot.launches_f)
        slot.busy = True
        flags = iter(slot.out_flags)

        def hand_out(t: torch.Tensor) -> torch.Tensor:
            c = t.detach().clone()
            return c.requires_grad_(True) if next(flags) else c
        return pt.tree_map_tensors(hand_out, slot.static_out), slot

    def _capture(self, slot: _Slot, leaves: List[Any], tpos: List[int], tree: Any, wrapped: bool, segs: int) -> None:
        from ..ops import bn as _bn
        static_in = [l.detach().clone().requires_grad_(l.requires_grad) if isinstance(l, torch.Tensor) else l
                     for l in leaves]
        x = pt.unflatten(static_in, tree, wrapped)
        pool = torch.cuda.graph_pool_handle()
        n0 = _f.LAUNCHES

        def run_forward():
            with torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.autocast, cache_enabled=False), \
                    _bn.segments(segs):
                return self.module(x)
        fwd = torch.cuda.CUDAGraph()
        y = capture(fwd, self.stream, pool, run_forward)
        n1 = _f.LAUNCHES
        out_leaves = [l for l in pt.flatten(y)[0] if isinstance(l, torch.Tensor)]
        out_flags = [bool(l.requires_grad and l.dim() > 0) for l in out_leaves]
        diff_out = [l for l, f in zip(out_leaves, out_flags) if f]
        static_gout = [torch.zeros_like(l) for l in diff_out]
        gin_leaves = [static_in[i] for i in tpos if static_in[i].requires_grad]

        def run_backward():
            grads = torch.autograd.grad(diff_out, gin_leaves + self.params, static_gout, allow_unused=True)
            for p, g in zip(self.params, grads[len(gin_leaves):]):
                if g is not None:
                    p.grad.add_(g)
            return [g if g is not None else torch.zeros_like(l) for g, l in zip(grads, gin_leaves)]
        bwd = torch.cuda.CUDAGraph()
        static_gin = capture(bwd, self.stream, pool, run_backward) if diff_out else []
        n2 = _f.LAUNCHES
        # the capture executed nothing: the BatchNorm accumulators, the gradients and the counters are untouched
        slot.fwd, slot.bwd, slot.pool = fwd, (bwd if diff_out else None), pool
        slot.static_in, slot.tpos, slot.static_out, slot.out_flags = static_in, tpos, y, out_flags
        slot.static_gout, slot.static_gin = static_gout, static_gin
        slot.launches_f, slot.launches_b = n1 - n0, n2 - n1
        _f.LAUNCHES = n0

    # -- backward ------------------------------------------------------------------------------------
    def backward(self, slot: _Slot, grads: List[torch.Tensor]) -> List[torch.Tensor]:
        """Replay the slot's backward with ``grads`` (one per differentiable output, in output order); returns the
        gradients of the stage inputs that asked for one, in input order."""
        assert slot.busy and len(grads) == len(slot.static_gout)
        with torch.no_grad():
            for s, g in zip(slot.static_gout, grads):
                s.copy_(g)
            if slot.bwd is not None:
                slot.bwd.replay()
                _f._count(slot.launches_b)
            out = [g.clone() for g in slot.static_gin]
        slot.busy = False
        return out
