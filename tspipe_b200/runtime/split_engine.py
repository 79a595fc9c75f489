"""Split placement: the teacher pipeline and the student pipeline live on different GPUs.

The reference always puts teacher stage ``j`` and student stage ``j`` on GPU ``j``
(`tspipe/gpu_worker.py:393-395`).  For distillation with a large forward-only teacher that wastes the
teacher's memory headroom on every student GPU; here ``runtime.placement: split`` gives the first
``len(model_split.target)`` ranks of a replica to the teacher stages and the remaining
``len(model_split.online)`` ranks to the student stages (supervised mode with a frozen teacher, or two-view
self-supervised mode with a momentum teacher):

* teacher ranks run ``T(b)`` microbatch by microbatch, as far ahead of the student as the output ring
  allows (``runtime.teacher_slots`` batches);
* student ranks run ``O(b)`` for all microbatches, the loss on the last student rank, ``B(b)`` in
  reverse order and ``OPT(b)``;
* the teacher's outputs never travel as messages on CUDA: the last teacher rank writes each microbatch's
  logits into a ring buffer in its own memory that is peer-mapped into the loss rank, and the fused KD
  loss kernel reads the teacher logits straight over NVLink (:class:`PeerMatrix`).  Two one-element
  token links order "slot filled" and "slot free" between the two ranks.  On CPU / gloo the logits are
  sent over the token link instead;
* a momentum teacher (BYOL / MoCo): after ``OPT(k)`` every student rank packs the parameter runs each teacher
  stage needs (:func:`tspipe_b200.runtime.ema_plan.split_placement_routes`) and sends them over a link of its own
  (peer memory + copy engine on CUDA); a teacher rank applies update ``k`` before its first forward of batch
  ``k + 2``, which is the one-step-stale teacher of the interleaved schedule (``T(b+1)`` sits between ``OPT(b-1)``
  and ``OPT(b)`` there).  The teacher therefore runs at most two batches ahead of the student's optimizer.  Both
  networks see both views of every microbatch; the loss rank copies the teacher's outputs of a batch out of the
  peer-mapped ring with the copy engine.
"""
from __future__ import annotations

import contextlib
import queue
import threading
import time
import traceback
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..batch_ops import Batch, ScatterGatherFn, defaultScatterGatherFn
from ..comm.links import Link, MetaBoard
from ..comm.peer import PeerView
from ..logger import Log
from ..utils import pytree as pt
from .engine import EngineError, FeedMsg, FlushMsg, StopMsg, _rebuild
from .state import FlatParams


class PeerMatrix(PeerView):
    """A ``[rows, cols]`` matrix in another GPU's memory (row-major), usable as the teacher operand of the
    fused loss kernels."""
    is_cuda = True

    def __init__(self, view: PeerView, rows: int, cols: int):
        super().__init__(view.data_ptr(), rows * cols, view.dtype, view.owner_rank, view)
        self.shape = (rows, cols)

    def detach(self) -> "PeerMatrix":
        return self


class SplitTopology:
    """Per-replica layout ``[teacher stages | student stages]`` and its process groups."""
    _instances = 0

    def __init__(self, pt_: int, ps: int, dp: int, device: torch.device, timeout_s: float = 600.0,
                 ema_pairs: bool = False):
        import datetime
        self.pt, self.ps, self.dp, self.device = pt_, ps, dp, device
        self.ema_groups: Dict[Any, Any] = {}          # (teacher stage, student stage) -> two-rank group
        self.pp = pt_ + ps
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        if self.pp * dp != self.world:
            raise ValueError(f"world size {self.world} != dp {dp} x (teacher {pt_} + student {ps})")
        self.replica, self.local = self.rank // self.pp, self.rank % self.pp
        self.is_teacher = self.local < pt_
        self.stage = self.local if self.is_teacher else self.local - pt_
        self.n_stage = pt_ if self.is_teacher else ps
        self.is_first, self.is_last = self.stage == 0, self.stage == self.n_stage - 1
        to = datetime.timedelta(seconds=timeout_s)
        self.fwd: Dict[int, Any] = {}
        self.bwd: Dict[int, Any] = {}
        self.tok_fill = self.tok_free = self.pair_group = None
        for r in range(dp):
            base = r * self.pp
            for chain_lo, n in ((0, pt_), (pt_, ps)):
                for j in range(n - 1):
                    pair = [base + chain_lo + j, base + chain_lo + j + 1]
                    gf, gb = dist.new_group(ranks=pair, timeout=to), dist.new_group(ranks=pair, timeout=to)
                    if self.rank in pair:
                        self.fwd[pair[0]], self.bwd[pair[0]] = gf, gb
            if ema_pairs:                                        # student stage -> teacher stage parameter links
                for jt in range(pt_):
                    for js in range(ps):
                        pair = [base + jt, base + pt_ + js]
                        g = dist.new_group(ranks=pair, timeout=to)
                        if self.rank in pair:
                            self.ema_groups[(jt, js)] = g
            pair = [base + pt_ - 1, base + self.pp - 1]          # last teacher rank, loss rank
            g1, g2, g3 = (dist.new_group(ranks=pair, timeout=to) for _ in range(3))
            if self.rank in pair:
                self.tok_fill, self.tok_free, self.pair_group, self.pair = g1, g2, g3, pair
        self.dp_group = None
        if dp > 1:
            for l in range(self.pp):
                ranks = [r * self.pp + l for r in range(dp)]
                g = dist.new_group(ranks=ranks, timeout=to)
                if self.rank in ranks:
                    self.dp_group = g
        from torch.distributed.distributed_c10d import _get_default_store
        SplitTopology._instances += 1       # every pipeline of a job gets its own key space in the store
        self.store = dist.PrefixStore(f"tspipe_split_ctl{SplitTopology._instances}", _get_default_store())

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"

    @property
    def is_loss_rank(self) -> bool:
        return (not self.is_teacher) and self.is_last

    @property
    def is_teacher_out_rank(self) -> bool:
        return self.is_teacher and self.is_last


class SplitKDEngine:
    def __init__(self, topo: SplitTopology, config: Dict[str, Any], partition: nn.Module,
                 optimizer: Optional[torch.optim.Optimizer], loss_fn: Callable, target_train_mode: bool = False,
                 scatter_gather_fn: ScatterGatherFn = defaultScatterGatherFn, args: Any = None, extra_args: Any = None,
                 inbox=None, ssl: bool = False, momentum: float = 1.0, ema_routes=None):
        self.topo, self.cfg, self.module = topo, config, partition
        # two-view self-supervised mode: both nets see views 0 and 1; supervised: student view 0, teacher view 1
        self.ssl = bool(ssl)
        self.views_s, self.views_t = ((0, 1), (0, 1)) if self.ssl else ((0,), (1,))
        self.optimizer, self.loss_fn, self.sg = optimizer, loss_fn, scatter_gather_fn
        self.args, self.extra_args = args, extra_args
        self.device, self.cuda = topo.device, topo.is_cuda
        rt = config["runtime"]
        self.U = int(rt["num_ubatch"] or max(topo.ps - 1, 1))
        self.autocast = rt["dtype"] == "bf16"
        self.fused = bool(rt["fused"]) and self.cuda
        self.slots = int(rt.get("teacher_slots", 2))
        self.peer = self.cuda and bool(rt.get("peer_memory", True))
        self.inbox = inbox if inbox is not None else queue.Queue()
        self.module.to(self.device)
        if topo.is_teacher:
            self.module.train(target_train_mode)
            for p in self.module.parameters():
                p.requires_grad_(False)
            self.flat = FlatParams(list(self.module.parameters()), self.device, with_grad=False) \
                if ema_routes is not None else None
        else:
            self.module.train()
            self.flat = FlatParams(list(self.module.parameters()), self.device, with_grad=True)
            if optimizer is not None and hasattr(optimizer, "bind_flat"):
                optimizer.bind_flat(self.flat, use_kernel=self.fused)
        self.compute = torch.cuda.Stream(self.device) if self.cuda else None
        base = topo.replica * topo.pp + (0 if topo.is_teacher else topo.pt)
        me = topo.rank
        from ..comm.peer_link import make_link
        peer_links = self.cuda and bool(rt.get("peer_links", True)) and bool(rt.get("peer_memory", True))
        if self.fused:
            # the one-thread ordering kernels of the peer-memory links (or the library's send / receive kernels) must
            # not queue behind a persistent GEMM that fills every SM
            from ..ops import fused as _fused
            reserve = rt.get("sm_reserve")
            _fused.set_sm_reserve(int(reserve) if reserve is not None else (4 if peer_links else 8))

        def link(group, peer_rank: int, tag: str):
            # peer memory + copy engines between GPUs of this node, the torch.distributed link otherwise; the name is
            # the same on both ends (boundaries are numbered by their lower rank)
            peer_dev = (self.device.index + peer_rank - me) if self.cuda else None
            if peer_dev is not None and not 0 <= peer_dev < torch.cuda.device_count():
                peer_dev = None
            return make_link(group, peer_rank, self.device, store=topo.store, name=f"plink/split/{tag}",
                             peer_device=peer_dev, use_peer=peer_links,
                             limit_ms=int(min(max(float(rt["timeout_s"]), 1.0), 600.0) * 1000))

        # stage boundaries inside the two chains: torch.distributed links
        self.fwd_in = Link(topo.fwd[me - 1], me - 1, self.device) if not topo.is_first else None
        self.fwd_out = Link(topo.fwd[me], me + 1, self.device) if not topo.is_last else None
        self.bwd_in = Link(topo.bwd[me], me + 1, self.device) if (not topo.is_teacher and not topo.is_last) else None
        self.bwd_out = Link(topo.bwd[me - 1], me - 1, self.device) if (not topo.is_teacher and not topo.is_first) else None
        other = None
        self.fill_link = self.free_link = None
        if topo.is_teacher_out_rank or topo.is_loss_rank:
            other = topo.pair[1] if topo.is_teacher_out_rank else topo.pair[0]
            # "slot filled" / "slot free" tokens.  A library receive for a token stays resident on the GPU until the
            # token comes (a whole batch later), in the way of every persistent GEMM launched meanwhile, so with a
            # frozen teacher the tokens go over peer-memory links.  With a momentum teacher they stay on the library:
            # a peer link's first send waits on the host for the receiver's first post, the teacher posts its first
            # "free" receive only at batch 3, which needs the student's parameters of step 1, which the student
            # sends only after that first "free" send has returned.
            if ema_routes is None:
                self.fill_link = link(topo.tok_fill, other, f"fill{topo.pair[0]}")
                self.free_link = link(topo.tok_free, other, f"free{topo.pair[0]}")
            else:
                self.fill_link = Link(topo.tok_fill, other, self.device)
                self.free_link = Link(topo.tok_free, other, self.device)
        self.meta = MetaBoard(topo.store, topo.replica)
        self.ring: Optional[List[torch.Tensor]] = None
        self.ring_views: Optional[List[Any]] = None
        self.feeds: Dict[int, FeedMsg] = {}
        self.highest_fed, self.last_batch, self._flushing = 0, None, False
        self.losses: "queue.Queue" = queue.Queue()
        self.error: Optional[BaseException] = None
        self.thread: Optional[threading.Thread] = None
        self.on_batch_done: Optional[Callable[[int], None]] = None
        self.on_flushed: Optional[Callable[[int], None]] = None
        self.momentum, self.ga_count, self.op_count = float(momentum), 0, 0
        self._momentum_at: Dict[int, float] = {}          # batch -> momentum in force at its optimizer step
        self.ema_applied = 0                              # teacher rank: student steps folded into the teacher so far
        self.ema_in: Dict[int, Any] = {}                  # teacher rank: student stage -> link
        self.ema_out: Dict[int, Any] = {}                 # student rank: teacher stage -> link
        self.ema_sources = self.ema_dests = None
        if ema_routes is not None:
            from ..comm.peer_link import make_link
            sources, dests = ema_routes
            base_rank = topo.replica * topo.pp
            use_peer = self.cuda and bool(rt.get("peer_links", True)) and bool(rt.get("peer_memory", True))

            def ema_link(jt: int, js: int):
                peer_rank = base_rank + (topo.pt + js if topo.is_teacher else jt)
                peer_dev = (self.device.index + peer_rank - topo.rank) if self.cuda else None
                if peer_dev is not None and not 0 <= peer_dev < torch.cuda.device_count():
                    peer_dev = None
                return make_link(topo.ema_groups[(jt, js)], peer_rank, self.device, store=topo.store,
                                 name=f"plink/r{topo.replica}/ema{js}to{jt}", peer_device=peer_dev, use_peer=use_peer,
                                 limit_ms=int(min(max(float(rt["timeout_s"]), 1.0), 600.0) * 1000))
            if topo.is_teacher:
                self.ema_sources = sources[topo.stage]
                self.ema_in = {js: ema_link(topo.stage, js) for js in sorted(self.ema_sources)}
            else:
                self.ema_dests = dests[topo.stage]
                self.ema_out = {jt: ema_link(jt, topo.stage) for jt in sorted(self.ema_dests)}
        self.online = self.module if not topo.is_teacher else nn.Sequential()
        self.target = self.module if topo.is_teacher else nn.Sequential()
        self.dp_fused = False
        self._warm()

    # -- plumbing -----------------------------------------------------------------------------------
    def _warm(self) -> None:
        t = self.topo
        links = sorted(set(list(t.fwd.items()) + [(k + 10 ** 6, v) for k, v in t.bwd.items()]), key=lambda kv: kv[0])
        for key, g in links:
            lo = key % 10 ** 6
            down = key < 10 ** 6
            src, dst = (lo, lo + 1) if down else (lo + 1, lo)
            mine = ((self.fwd_out if down else self.bwd_in) if t.rank == lo else (self.fwd_in if down else self.bwd_out))
            if not isinstance(mine, Link):
                continue                                # a peer-memory link (or none): no communicator behind it
            x = torch.zeros(1, device=self.device)
            (dist.send(x, dst, group=g) if t.rank == src else dist.recv(x, src, group=g))
        if t.tok_fill is not None and isinstance(self.fill_link, Link):
            a, b = t.pair
            x = torch.zeros(1, device=self.device)
            (dist.send(x, b, group=t.tok_fill) if t.rank == a else dist.recv(x, a, group=t.tok_fill))
            (dist.send(x, a, group=t.tok_free) if t.rank == b else dist.recv(x, b, group=t.tok_free))
        base_rank = t.replica * t.pp
        for (jt, js), g in sorted(t.ema_groups.items()):
            mine = self.ema_in.get(js) if t.is_teacher else self.ema_out.get(jt)
            if isinstance(mine, Link):                  # student -> teacher, one message to create the communicator
                x = torch.zeros(1, device=self.device)
                (dist.recv(x, base_rank + t.pt + js, group=g) if t.is_teacher else dist.send(x, base_rank + jt, group=g))
        if self.cuda:
            torch.cuda.synchronize(self.device)

    def _on_compute(self):
        return torch.cuda.stream(self.compute) if self.cuda else contextlib.nullcontext()

    def _amp(self):
        return torch.autocast(device_type=self.device.type, dtype=torch.bfloat16) if self.autocast \
            else contextlib.nullcontext()

    def start(self) -> None:
        self.thread = threading.Thread(target=self._guarded, name=f"tspipe-split-{self.topo.rank}", daemon=True)
        self.thread.start()

    def join(self, timeout: Optional[float] = None) -> None:
        if self.thread is not None:
            self.thread.join(timeout)
        if self.error is not None:
            raise EngineError(f"split engine on rank {self.topo.rank} failed") from self.error

    def _guarded(self) -> None:
        try:
            self.run()
        except BaseException as e:  # noqa: BLE001
            self.error = e
            Log.e(f"rank {self.topo.rank} split executor died:\n{traceback.format_exc()}")
            self.losses.put((-1, e))
            try:
                self.topo.store.set(f"dead/{self.topo.rank}", repr(e).encode()[:2000])
            except Exception:
                pass

    def _pump(self, block: bool) -> bool:
        try:
            msg = self.inbox.get(timeout=0.2) if block else self.inbox.get_nowait()
        except queue.Empty:
            return False
        if isinstance(msg, StopMsg):
            self.last_batch, self._flushing = msg.last_batch, False
        elif isinstance(msg, FlushMsg):
            self.last_batch, self._flushing = msg.last_batch, True
        elif isinstance(msg, FeedMsg):
            self.feeds[msg.batch_id] = msg
            self.highest_fed = max(self.highest_fed, msg.batch_id)
        return True

    def _have_batch(self, b: int) -> bool:
        deadline = time.monotonic() + float(self.cfg["runtime"]["timeout_s"])
        while True:
            if b <= self.highest_fed:
                return True
            if self.last_batch is not None and b > self.last_batch:
                return False
            if self.error is not None:
                raise EngineError("stopping: failure reported") from self.error
            if not self._pump(True) and time.monotonic() > deadline:
                raise EngineError(f"rank {self.topo.rank}: no batch {b} and no stop within the timeout")

    # -- main loop ----------------------------------------------------------------------------------
    def run(self) -> None:
        b = 1
        while True:
            if not self._have_batch(b):
                self._drain(b - 1)
                if not self._flushing:
                    return
                self._flushing, self.last_batch = False, None
                if self.on_flushed is not None:
                    self.on_flushed(b - 1)
                continue
            if self.topo.is_teacher:
                self._teacher_batch(b)
            else:
                self._student_batch(b)
            self.feeds.pop(b - 1, None)
            if self.on_batch_done is not None:
                self.on_batch_done(b)
            b += 1

    def _input(self, b: int, u: int, view: int) -> Any:
        msg = self.feeds[b]
        cache = msg.__dict__.setdefault("_scattered", {})
        if view not in cache:
            cache[view] = self.sg.scatter(msg.views[view], self.U)
        ub = cache[view][u]
        data = ub.value if isinstance(ub, Batch) else ub
        if self.cuda:
            if msg.ready_event is not None:
                torch.cuda.current_stream().wait_event(msg.ready_event)
            data = pt.tree_map_tensors(lambda t: t if t.is_cuda else t.to(self.device, non_blocking=True), data)
        return data

    def _recv(self, net: str, b: int):
        meta = self.meta.fetch(f"s{self.topo.rank - 1}", net, b)
        specs, tree, wrapped, others = meta[0]
        h = self.fwd_in.post_recv([(sh, dt) for sh, dt, _ in specs])
        return _rebuild(h.wait(), others, tree, wrapped), [rg for _, _, rg in specs]

    def _send(self, net: str, b: int, y: Any) -> None:
        leaves, tree, wrapped = pt.flatten(y)
        ts = [l.detach() for l in leaves if isinstance(l, torch.Tensor)]
        rgs = [bool(l.requires_grad and l.dim() > 0) for l in leaves if isinstance(l, torch.Tensor)]
        others = [(i, l) for i, l in enumerate(leaves) if not isinstance(l, torch.Tensor)]
        self.meta.publish(f"s{self.topo.rank}", net, b, [([(tuple(t.shape), t.dtype, rg) for t, rg in zip(ts, rgs)],
                                                           tree, wrapped, others)])
        self.fwd_out.send(ts)

    # -- teacher side -------------------------------------------------------------------------------
    def _note_momentum(self, b: int) -> None:
        msg = self.feeds.get(b)
        if msg is not None and msg.new_momentum is not None:
            self.momentum = msg.new_momentum
        self._momentum_at[b] = self.momentum
        self._momentum_at.pop(b - 4, None)

    @torch.no_grad()
    def _apply_teacher_updates(self, upto: int) -> None:
        """Teacher rank: fold the student's steps ``ema_applied + 1 .. upto`` into the teacher, one after the other,
        from the packed parameter runs the student ranks sent after each of those steps."""
        while self.ema_applied < upto:
            k = self.ema_applied + 1
            m = self._momentum_at.get(k, self.momentum)
            for js, runs in sorted(self.ema_sources.items()):
                total = sum(n for _, _, n in runs)
                buf = self.ema_in[js].post_recv([((total,), self.flat.data.dtype)]).wait()[0]
                pos = 0
                for t_off, _, n in runs:
                    dst, src = self.flat.data[t_off:t_off + n], buf[pos:pos + n]
                    if self.fused:
                        from ..ops import fused
                        fused.ema_update_(dst, src, m)
                    else:
                        dst.lerp_(src, 1.0 - m)
                    pos += n
            self.ema_applied = k

    def _send_student_params(self) -> None:
        """Student rank, after an optimizer step: a packed copy of the runs each teacher stage needs (the copy is
        the snapshot: later steps may overwrite the parameters while the message is still in flight)."""
        for jt, runs in sorted(self.ema_dests.items()):
            self.ema_out[jt].send([torch.cat([self.flat.data[o:o + n] for o, n in runs])])

    def _teacher_batch(self, b: int) -> None:
        t = self.topo
        self._note_momentum(b)
        with self._on_compute():
            if self.ema_sources is not None:
                self._apply_teacher_updates(b - 2)      # T(b) runs on the teacher after the student's step b - 2
            if t.is_last and self.peer and b > self.slots:
                self.free_link.post_recv([((1,), torch.float32)]).wait()      # slot of batch b - slots was consumed
            for u in range(self.U):
                for v in self.views_t:
                    x = self._input(b, u, v) if t.is_first else self._recv("t", b)[0]
                    with torch.no_grad(), self._amp():
                        y = self.module(x)
                    self.op_count += 1
                    if not t.is_last:
                        self._send("t", b, y)
                    else:
                        self._publish_teacher(b, u, pt.unwrap(y), self.views_t.index(v))
            if t.is_last and self.peer:
                self.fill_link.send([torch.ones(1, device=self.device)])      # all microbatches of b are in the ring

    def _publish_teacher(self, b: int, u: int, y: torch.Tensor, vi: int = 0) -> None:
        """Microbatch ``u`` of view number ``vi`` goes to rows ``(vi * U + u) * n ...`` of the batch's ring slot."""
        if not isinstance(y, torch.Tensor) or y.dim() != 2:
            raise EngineError("split placement expects the teacher to end in a [batch, classes] tensor")
        if not self.peer:
            self.fill_link.send([y.contiguous()])
            if b == 1 and u == 0:
                self.topo.store.set(f"tshape/{self.topo.replica}", repr((tuple(y.shape), str(y.dtype))).encode())
            return
        if self.ring is None:
            from ..comm import peer
            rows = y.shape[0] * self.U * len(self.views_t)
            self.ring = [torch.zeros(rows, y.shape[1], dtype=y.dtype, device=self.device) for _ in range(self.slots)]
            self.topo.store.set(f"tshape/{self.topo.replica}", repr((tuple(y.shape), str(y.dtype))).encode())
            self._ring_keep = [peer.exchange(r.view(-1), self.topo.pair_group, self.topo.pair) for r in self.ring]
        slot = self.ring[(b - 1) % self.slots]
        n = y.shape[0]
        row = (vi * self.U + u) * n
        slot[row:row + n].copy_(y)

    # -- student side -------------------------------------------------------------------------------
    def _student_batch(self, b: int) -> None:
        t = self.topo
        msg = self.feeds[b]
        acts = []
        self._note_momentum(b)
        with self._on_compute():
            for u, v in [(u, v) for u in range(self.U) for v in self.views_s]:
                if t.is_first:
                    x, gin = self._input(b, u, v), []
                    leaves = None
                else:
                    x, flags = self._recv("o", b)
                    leaves, tree, wrapped = pt.flatten(x)
                    pos = [i for i, l in enumerate(leaves) if isinstance(l, torch.Tensor)]
                    gin = [i for i, rg in zip(pos, flags) if rg]
                    for i in gin:
                        leaves[i] = leaves[i].detach().requires_grad_(True)
                    x = pt.unflatten(leaves, tree, wrapped)
                with self._amp():
                    y = self.module(x)
                self.op_count += 1
                acts.append((leaves, gin, y))
                if not t.is_last:
                    self._send("o", b, y)
            grads = self._loss(b, msg, [a[2] for a in acts]) if t.is_last else None
            for u in reversed(range(len(acts))):          # items in reverse forward order
                leaves, gin, y = acts[u]
                oleaves = pt.flatten(y)[0]
                outs = [l for l in oleaves if isinstance(l, torch.Tensor) and l.requires_grad and l.dim() > 0]
                if t.is_last:
                    g = grads[u]
                else:
                    g = self.bwd_in.post_recv([(tuple(o.shape), o.dtype) for o in outs]).wait()
                if outs:
                    torch.autograd.backward(outs, g)
                if not t.is_first:
                    self.bwd_out.send([leaves[i].grad if leaves[i].grad is not None else torch.zeros_like(leaves[i])
                                       for i in gin])
                acts[u] = None
            self._optimize(msg)

    def _teacher_outputs(self, b: int, rows: int):
        """Teacher logits of batch ``b`` on the loss rank: a :class:`PeerMatrix` over the teacher GPU's ring
        slot (CUDA), or the received tensors (CPU)."""
        import ast
        shape, dt = ast.literal_eval(self.topo.store.get(f"tshape/{self.topo.replica}").decode())
        dtype = getattr(torch, dt.split(".")[-1])
        nv = len(self.views_t)
        if not self.peer:
            parts = [self.fill_link.post_recv([(shape, dtype)]).wait()[0] for _ in range(self.U * nv)]
            if not self.ssl:
                return torch.cat(parts)
            return [torch.cat(parts[vi::nv]) for vi in range(nv)]          # sent microbatch by microbatch, views inside
        if self.ring_views is None:
            from ..comm import peer
            dummy = [torch.zeros(1, dtype=dtype, device=self.device) for _ in range(self.slots)]
            self._ring_keep = [peer.exchange(d, self.topo.pair_group, self.topo.pair) for d in dummy]
            self.ring_views = [k[0] for k in self._ring_keep]
        self.fill_link.post_recv([((1,), torch.float32)]).wait()
        view = self.ring_views[(b - 1) % self.slots]
        if self.ssl:
            # the generic two-view losses take tensors: bring the batch's slot over with the copy engine
            import ctypes as _c
            from ..ops import fused
            local = torch.empty(nv, shape[0] * self.U, shape[1], dtype=dtype, device=self.device)
            L = fused.lib()
            L.tsp_copy_async.restype = _c.c_int
            fused._check(L.tsp_copy_async(fused._ptr(local), _c.c_void_p(view.data_ptr()),
                                          _c.c_int64(local.numel() * local.element_size()), fused._stream()),
                         "tsp_copy_async")
            return [local[vi] for vi in range(nv)]
        full = PeerView(view.data_ptr(), shape[0] * self.U * shape[1], dtype, view.owner_rank, view)
        return PeerMatrix(full, shape[0] * self.U, shape[1])

    def _loss(self, b: int, msg: FeedMsg, outs: List[Any]) -> List[List[torch.Tensor]]:
        ys = [pt.unwrap(o) for o in outs]
        nv = len(self.views_s)
        # forward order is microbatch by microbatch with the views inside: view vi owns items vi, vi + nv, ...
        cats = [torch.cat([y.detach() for y in ys[vi::nv]]).requires_grad_(True) for vi in range(nv)]
        cat = cats[0]
        teacher = self._teacher_outputs(b, cat.shape[0])
        labels = msg.labels
        if self.cuda and labels is not None:
            labels = pt.tree_map_tensors(lambda t: t if t.is_cuda else t.to(self.device, non_blocking=True), labels)
        with self._amp():
            if self.ssl:
                loss = self.loss_fn(cats[0], cats[1], teacher[0], teacher[1], self.args, self.extra_args)
            else:
                loss = self.loss_fn(cat, teacher, labels, self.args, self.extra_args, msg.epoch)
        if self.cuda:
            host = torch.empty((), dtype=torch.float32, pin_memory=True)
            host.copy_(loss.detach().float(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.losses.put((b, (host, ev)))
        else:
            self.losses.put((b, float(loss.detach())))
        torch.autograd.backward(loss)
        if self.peer:
            self.free_link.send([torch.ones(1, device=self.device)])          # the teacher slot may be reused
        per_view = [c.grad.split([y.shape[0] for y in ys[vi::nv]]) for vi, c in enumerate(cats)]
        return [[per_view[i % nv][i // nv]] for i in range(len(ys))]

    def _optimize(self, msg: FeedMsg) -> None:
        if msg.new_lr is not None and self.optimizer is not None:
            lrs = msg.new_lr if isinstance(msg.new_lr, (list, tuple)) else [msg.new_lr] * len(self.optimizer.param_groups)
            for g, lr in zip(self.optimizer.param_groups, lrs):
                g["lr"] = lr
        self.flat.collect_stray_grads()
        if self.topo.dp_group is not None:
            dist.all_reduce(self.flat.grad, group=self.topo.dp_group)
            self.flat.grad.div_(self.topo.dp)
        if self.optimizer is not None:
            self.optimizer.step()
        self.flat.zero_grad()
        if self.ema_dests is not None:
            self._send_student_params()
        if self.cuda:
            from ..ops import conv as _conv
            from ..ops import gemm as _gemm
            _conv.clear_weight_cache()              # bf16 weight copies of the tcgen05 convolutions and linears
            _gemm.clear_weight_cache()

    def _drain(self, done: int = 0) -> None:
        if self.topo.is_teacher and self.ema_sources is not None:
            with self._on_compute():
                self._apply_teacher_updates(done)       # the student's last two steps are still on their way
        for link in [self.fwd_out, self.bwd_out, self.fill_link, self.free_link] + list(self.ema_out.values()):
            if link is not None:
                link.flush()
        if self.cuda:
            self.compute.synchronize()
