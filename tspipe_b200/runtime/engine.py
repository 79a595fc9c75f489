"""Per-rank stage engine: one executor walking its own column of the schedule.

What the reference spreads over seven role threads, a condition variable, eleven task types
with spin-checked preconditions and ~5 host synchronisations per microbatch
(`tspipe/gpu_worker.py:26-149,357-381,468-563`, `tspipe/gpu_task.py:89-834`) is here ONE
loop per rank over :func:`tspipe_b200.schedule.batch_block`:

* ``T`` / ``O``  forward one microbatch through the teacher / student partition
  (`gpu_task.py:431-530`), input from the feeder (stage 0) or the upstream link, output to the
  downstream link or the loss collector (last stage);
* ``LOSS``      full-batch loss on the last stage and per-nano-batch output gradients
  (`gpu_task.py:89-226`);
* ``B``         backward of one nano-batch, input gradient to the upstream link
  (`gpu_task.py:229-285`);
* ``OPT``       data-parallel gradient sync, optimizer step, momentum-teacher update
  (`gpu_task.py:322-417`).

Ordering between compute, copies and transfers is expressed with CUDA streams and events
only; the host never waits for the device except when the caller asks for a loss value.
On CPU (gloo) the same loop runs with blocking transfers.
"""
from __future__ import annotations

import contextlib
import queue
import threading
import time
import traceback
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import nn

from ..batch_ops import Batch, ScatterGatherFn, defaultScatterGatherFn
from ..comm.links import Link, MetaBoard, RecvHandle
from ..comm.peer_link import make_link
from ..comm.topology import Topology
from ..logger import Log
from ..schedule import Op, OpKind, ScheduleSpec, batch_block
from ..utils import pytree as pt
from .state import FlatParams, corresponding_prefix


# ---------------------------------------------------------------------------------------------
# messages from the feeder (same process: queue.Queue; spawned worker: multiprocessing queue)
# ---------------------------------------------------------------------------------------------
@dataclass
class FeedMsg:
    batch_id: int
    views: Optional[List[Any]] = None          # [view_1, view_2] mini-batch data (stage 0 only)
    labels: Any = None                         # last stage only (KD mode)
    new_lr: Any = None                         # scalar or per-group list, applied at OPT(batch_id)
    new_momentum: Optional[float] = None
    force_step: bool = False                   # epoch boundary: step even if accumulation is incomplete
    epoch: int = 0
    ready_event: Any = None                    # CUDA event: device copies of `views` are complete


@dataclass
class StopMsg:
    last_batch: int


@dataclass
class FlushMsg:
    """Finish every batch up to ``last_batch`` without look-ahead, then wait for more feeds; the next
    batch refills the pipeline."""
    last_batch: int


@dataclass
class EpochMsg:
    batch_id: int                              # the optimizer steps at this batch regardless of accumulation


class EngineError(RuntimeError):
    pass


# ---------------------------------------------------------------------------------------------
# teacher update strategies
# ---------------------------------------------------------------------------------------------
class TeacherUpdater:
    def step(self, momentum: float) -> None:
        raise NotImplementedError


class FrozenTeacher(TeacherUpdater):
    def step(self, momentum: float) -> None:
        return


class CallbackTeacher(TeacherUpdater):
    """The reference contract: ``fn(momentum, online_new_params, target_prev_params) -> list``
    evaluated per partition (`gpu_task.py:403-406`), result copied into the live teacher."""

    def __init__(self, fn: Callable, online: Sequence[nn.Parameter], target: Sequence[nn.Parameter]):
        self.fn, self.online, self.target = fn, list(online), list(target)

    @torch.no_grad()
    def step(self, momentum: float) -> None:
        new = self.fn(momentum, [p.detach() for p in self.online], [p for p in self.target])
        for p, q in zip(self.target, new):
            if q is not p:
                p.copy_(q)


class FlatEmaTeacher(TeacherUpdater):
    """``t = m*t + (1-m)*s`` over flat buffers in one launch (CUDA: the sm_100a kernel, which
    may read ``s`` through a peer pointer; CPU: one ``lerp_``)."""

    def __init__(self, teacher: FlatParams, student_flat: torch.Tensor, segments=None, use_kernel: bool = False):
        self.teacher, self.student_flat, self.segments, self.use_kernel = teacher, student_flat, segments, use_kernel

    @torch.no_grad()
    def step(self, momentum: float) -> None:
        n = self.teacher.total
        if self.use_kernel:
            from ..ops import fused
            fused.ema_update_(self.teacher.data, self.student_flat[:n], momentum)
        else:
            self.teacher.data.lerp_(self.student_flat[:n], 1.0 - momentum)


class OptimizerFusedEma(TeacherUpdater):
    """The momentum update rides in the optimizer's own launch (:mod:`tspipe_b200.optim.flat`):
    the freshly written student value is blended into the local teacher buffer before it leaves
    the registers, so the step touches the teacher once and the student not at all again."""

    def __init__(self, optimizer, teacher: FlatParams):
        self.optimizer = optimizer
        optimizer.teacher_flat = teacher.data

    def before_step(self, momentum: float) -> None:
        self.optimizer.ema_momentum = momentum

    def step(self, momentum: float) -> None:
        return


class CrossStageEmaTeacher(TeacherUpdater):
    """Momentum update when teacher and student are cut at different children: some of a teacher
    stage's student counterparts live on other ranks (:mod:`tspipe_b200.runtime.ema_plan`).

    Transfer path (any backend): every stage packs the runs other stages need, all exchanges of
    the step go out as one batched point-to-point group on the replica's pipeline group, then the
    runs are blended in.  Peer path (CUDA, same node): the student buffers are mapped into every
    rank (:mod:`tspipe_b200.comm.peer`) and the sm_100a kernel reads the remote runs straight
    over NVLink; the batched exchange then only carries one-element "my step is done" tokens."""

    def __init__(self, topo: Topology, plan, teacher: FlatParams, student: FlatParams, peer_flats=None,
                 use_kernel: bool = False):
        self.topo, self.plan, self.teacher, self.student = topo, plan, teacher, student
        self.peer_flats, self.use_kernel = peer_flats, use_kernel
        self._seg_cache = None

    def _rank(self, stage: int) -> int:
        return self.topo.rank_of(self.topo.replica, stage)

    @torch.no_grad()
    def step(self, momentum: float) -> None:
        plan, t, s = self.plan, self.teacher.data, self.student.data
        peer = self.peer_flats is not None
        ops, recv_bufs = [], {}
        for dst, runs in sorted(plan.send.items()):
            buf = s.new_zeros(1) if peer else torch.cat([s[o:o + n] for o, n in runs])
            ops.append(dist.P2POp(dist.isend, buf, self._rank(dst), group=self.topo.pp_group))
        for src, runs in sorted(plan.recv.items()):
            buf = s.new_empty(1 if peer else sum(n for _, _, n in runs))
            recv_bufs[src] = buf
            ops.append(dist.P2POp(dist.irecv, buf, self._rank(src), group=self.topo.pp_group))
        works = dist.batch_isend_irecv(ops) if ops else []
        for t_off, s_off, n in plan.local:
            self._blend(t[t_off:t_off + n], s[s_off:s_off + n], momentum)
        for w in works:
            w.wait()
        for src, runs in sorted(plan.recv.items()):
            pos = 0
            for t_off, s_off, n in runs:
                if peer:
                    self._blend(t[t_off:t_off + n], self.peer_flats[src][s_off:s_off + n], momentum)
                else:
                    self._blend(t[t_off:t_off + n], recv_bufs[src][pos:pos + n], momentum)
                pos += n

    def _blend(self, t: torch.Tensor, s: torch.Tensor, momentum: float) -> None:
        if self.use_kernel:
            from ..ops import fused
            fused.ema_update_(t, s, momentum)
        else:
            t.lerp_(s, 1.0 - momentum)


# ---------------------------------------------------------------------------------------------
@dataclass
class _Stored:
    inputs: List[Any]                 # per nano: flat input leaves (leaf tensors requiring grad kept here)
    outputs: List[Any]                # per nano: flat output leaves (with graph)
    grad_in_idx: List[int]            # indices of input leaves that carry a gradient upstream
    grad_out_idx: List[int]           # indices of output leaves that require grad
    graph: Any = None                 # the CUDA-graph slot that ran the forward (its backward is a replay too)


class StageEngine:
    def __init__(self, topo: Topology, config: Dict[str, Any], partition_online: nn.Module,
                 partition_target: nn.Module, optimizer: Optional[torch.optim.Optimizer],
                 loss_fn: Callable, target_update_fn: Optional[Callable], momentum: float,
                 kd_mode: bool, target_train_mode: bool = True,
                 scatter_gather_fn: ScatterGatherFn = defaultScatterGatherFn,
                 args: Any = None, extra_args: Any = None, inbox=None, profiler=None, ema_plan=None):
        self.topo, self.cfg = topo, config
        self.device = topo.device
        self.cuda = topo.is_cuda
        self.online, self.target = partition_online, partition_target
        self.optimizer, self.loss_fn, self.momentum = optimizer, loss_fn, momentum
        self.kd = kd_mode
        self.sg = scatter_gather_fn
        self.args, self.extra_args = args, extra_args
        self.inbox = inbox if inbox is not None else queue.Queue()
        self.profiler = profiler
        rt = config["runtime"]
        gp = config["gpipe_emulation"]
        n_ub = gp["num_ubatch"] if gp["enabled"] else rt["num_ubatch"]
        self.spec = ScheduleSpec(n_stages=topo.pp, n_ubatch=n_ub, bwd_split=rt["bwd_split"], kd=kd_mode,
                                 skip_staleness=config["optimizer"]["num_skip_initial_staleness"],
                                 gpipe=gp["enabled"])
        self.U, self.S = self.spec.n_ubatch, self.spec.bwd_split
        self.ga = max(int(config["optimizer"]["gradient_accumulation"]), 1)
        self.skip_optimizer = bool(config["optimizer"]["skip_optimizer"])
        self.autocast = rt["dtype"] == "bf16"
        self.fused = bool(rt["fused"]) and self.cuda
        self.channels_last = bool(rt["channels_last"])
        if self.cuda:
            from ..ops import bn as _bn
            _bn.set_enabled(self.fused)
            if self.fused:
                from ..ops import fused as _fused
                reserve = rt.get("sm_reserve")
                if reserve is None:
                    # kernels of the stage links must not queue behind a persistent kernel that fills every SM:
                    # the library's send / receive kernels, or the one-thread ordering kernels of the peer-memory
                    # links (their bytes move by copy engine, but a signal that waits for a whole convolution to
                    # finish adds its latency to every hop of the pipeline)
                    peer_links = bool(rt.get("peer_links", True)) and bool(rt.get("peer_memory", True))
                    reserve = (4 if peer_links else 8) if topo.pp > 1 else 0
                _fused.set_sm_reserve(int(reserve))

        self.online.to(self.device)
        self.target.to(self.device)
        if self.channels_last:
            self.online.to(memory_format=torch.channels_last)
            self.target.to(memory_format=torch.channels_last)
        if self.fused:
            from .fuse import fuse_partition
            self.online, self.target = fuse_partition(self.online), fuse_partition(self.target)
        self.online.train()
        self.target.train(target_train_mode)
        for p in self.target.parameters():
            p.requires_grad_(False)
        from ..batchnorm import BatchNormGroup
        self.bn_group_online = BatchNormGroup(self.online)
        self.bn_group_target = BatchNormGroup(self.target)
        self.merge_views = self._can_merge_views(rt)

        # flat state ---------------------------------------------------------------------------
        self.flat_online = FlatParams([p for p in self.online.parameters()], self.device, with_grad=True,
                                      pad_to=max(topo.dp, 1))
        self.flat_target = FlatParams([p for p in self.target.parameters()], self.device, with_grad=False)
        self._bind_optimizer()
        self.dp_fused = False
        self.dp_signals = None
        self._dp_event = None
        self._enable_dp_fused()
        self.ema_plan = ema_plan
        self.updater = self._make_updater(target_update_fn)

        # streams / links ------------------------------------------------------------------------
        if self.cuda:
            self.compute = torch.cuda.Stream(self.device)
            self.copy_stream = torch.cuda.Stream(self.device)
            self.dp_stream = torch.cuda.Stream(self.device)
        else:
            self.compute = self.copy_stream = self.dp_stream = None
        j = topo.stage
        rt = self.cfg["runtime"]

        def link(groups, boundary: int, peer_rank: int, tag: str):
            # activations and gradients cross a stage boundary through peer memory (copy engines) when both GPUs are
            # in this node; the torch.distributed link otherwise
            peer_dev = (self.device.index + peer_rank - topo.rank) if self.cuda else None
            if peer_dev is not None and not 0 <= peer_dev < torch.cuda.device_count():
                peer_dev = None
            return make_link(groups[boundary], peer_rank, self.device, store=topo.store,
                             name=f"plink/r{topo.replica}/{tag}{boundary}", peer_device=peer_dev,
                             use_peer=bool(rt.get("peer_links", True)) and bool(rt.get("peer_memory", True)),
                             slots=int(rt.get("link_slots", 4)), channels_last=self.channels_last and self.cuda,
                             limit_ms=int(min(max(float(rt["timeout_s"]), 1.0), 600.0) * 1000))

        self.fwd_in = link(topo.fwd_groups, j - 1, topo.prev_rank, "f") if not topo.is_first else None
        self.bwd_out = link(topo.bwd_groups, j - 1, topo.prev_rank, "b") if not topo.is_first else None
        self.fwd_out = link(topo.fwd_groups, j, topo.next_rank, "f") if not topo.is_last else None
        self.bwd_in = link(topo.bwd_groups, j, topo.next_rank, "b") if not topo.is_last else None
        self.meta = MetaBoard(topo.store, topo.replica)

        # run-time state -------------------------------------------------------------------------
        self.feeds: Dict[int, FeedMsg] = {}
        self.last_batch: Optional[int] = None
        self.highest_fed = 0
        self.acts: Dict[Tuple[int, int, int], _Stored] = {}            # (batch, view, ub) -> student activations
        self.t_out: Dict[Tuple[int, int], List[Any]] = {}               # last stage: (batch, view) -> teacher outputs per ub
        self.o_out: Dict[Tuple[int, int], List[Any]] = {}               # last stage: student outputs (flat leaves per nano)
        self.out_grads: Dict[Tuple[int, int, int], List[torch.Tensor]] = {}   # last stage: (batch, view, nano) -> grads
        self.fwd_posted: Dict[Tuple, RecvHandle] = {}
        self.bwd_posted: Dict[Tuple, RecvHandle] = {}
        self._fwd_iter = self._fwd_keys()
        self._bwd_order: Dict[int, List[Op]] = {}
        self._fwd_peek: Optional[Op] = None
        self.ga_count = 0
        self.force_steps: set = set()
        self.fill_batches: set = {self.spec.skip_staleness + 1}
        self._flushing = False
        self.on_flushed: Optional[Callable[[int], None]] = None
        self.steps_done = 0
        self._teacher_graphs: Dict[Any, Any] = {}
        self._teacher_graph_launches: Dict[Any, int] = {}
        self._graph_stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.async_emu = bool(config["async_param_update_emulation"]["enabled"]) and not gp["enabled"]
        self._alt_params = None
        self._initial_params = self.flat_online.data.clone() if self.async_emu else None
        self.student_graphs = None
        if (self.cuda and self.cfg["runtime"].get("cuda_graphs", False) and self.S == 1 and not self.async_emu
                and self.cfg["runtime"].get("student_graphs", True) and self.flat_online.grad is not None):
            from .stage_graph import StudentStageGraphs
            self.student_graphs = StudentStageGraphs(self.online, self.flat_online, self.autocast, self.device)
        self.watchdog = None
        self._amp_open = False
        self.error: Optional[BaseException] = None
        self.thread: Optional[threading.Thread] = None
        self.losses: "queue.Queue[Tuple[int, Any]]" = queue.Queue()
        self.op_count = 0
        self._in_op = False
        self.on_batch_done: Optional[Callable[[int], None]] = None
        self.on_idle: Optional[Callable[[], None]] = None
        self._warm_links()

    # -- set-up helpers ----------------------------------------------------------------------------
    def _bind_optimizer(self) -> None:
        """Optimizers from :mod:`tspipe_b200.optim` step the flat buffers in one or two launches."""
        opt = self.optimizer
        if opt is not None and hasattr(opt, "bind_flat"):
            opt.bind_flat(self.flat_online, use_kernel=self.fused)

    def _enable_dp_fused(self) -> None:
        """With pipeline replicas on CUDA, let the flat optimizer do reduce-scatter + step + all-gather in
        its own kernels over peer-mapped gradient / parameter buffers instead of an NCCL all-reduce."""
        opt, topo = self.optimizer, self.topo
        if not (topo.dp > 1 and self.fused and self.cfg["runtime"].get("peer_memory", True)
                and hasattr(opt, "enable_dp") and type(opt).__name__ in ("LARS", "AdamW")):
            return
        from ..comm import peer
        self.nvls_capable = peer.multicast_supported(self.device.index)
        if topo.rank == 0:
            Log.i(f"NVLink multicast (NVLS) capability: {self.nvls_capable}; gradients move by peer loads / stores")
        grads = peer.exchange(self.flat_online.grad, topo.dp_group, topo.dp_ranks)
        params = peer.exchange(self.flat_online.data, topo.dp_group, topo.dp_ranks)
        opt.enable_dp(topo.dp_group, grads, params, topo.replica)
        if self.cfg["runtime"].get("dp_signals", True):
            # ordering between the replicas through signal words in peer memory (bounded device-side waits) instead
            # of tiny NCCL collectives; LARS exchanges its partial norms through peer stores as well
            from ..comm.signals import SignalPad
            limit_ms = int(min(max(float(self.cfg["runtime"]["timeout_s"]), 1.0), 120.0) * 1000)
            self.dp_signals = SignalPad(topo.dp_group, topo.dp_ranks, topo.replica, self.device, limit_ms=limit_ms)
            tables = None
            if type(opt).__name__ == "LARS":
                table = torch.zeros(topo.dp * 2 * max(len(self.flat_online.params), 1), dtype=torch.float32,
                                    device=self.device)
                tables = peer.exchange(table, topo.dp_group, topo.dp_ranks)
            opt.enable_signals(self.dp_signals, tables)
        self.dp_fused = True

    def _make_updater(self, fn: Optional[Callable]) -> TeacherUpdater:
        if fn is None:
            return FrozenTeacher()
        if getattr(fn, "is_ema", False):
            plan = self.ema_plan
            if plan is None or plan.is_local_prefix:
                if corresponding_prefix(self.flat_online, self.flat_target):
                    if hasattr(self.optimizer, "bind_flat") and self.cfg["runtime"].get("fuse_ema", True) \
                            and not self.dp_fused:
                        return OptimizerFusedEma(self.optimizer, self.flat_target)
                    return FlatEmaTeacher(self.flat_target, self.flat_online.data, use_kernel=self.fused)
            else:
                peers = None
                if self.cuda and self.cfg["runtime"].get("peer_memory", True) and (plan.recv or plan.send):
                    from ..comm import peer
                    peers = peer.share_over_group(self.flat_online, self.topo)
                return CrossStageEmaTeacher(self.topo, plan, self.flat_target, self.flat_online, peers,
                                            use_kernel=self.fused)
            fn = fn.reference_fn
        n = len(self.flat_target.params)
        return CallbackTeacher(fn, self.flat_online.params[:n], self.flat_target.params)

    def _warm_links(self) -> None:
        """Create every p2p communicator up front, boundary by boundary, in one global order."""
        for j in range(self.topo.pp - 1):
            for groups, down in ((self.topo.fwd_groups, True), (self.topo.bwd_groups, False)):
                if j not in groups:
                    continue
                lo, hi = self.topo.rank_of(self.topo.replica, j), self.topo.rank_of(self.topo.replica, j + 1)
                src, dst = (lo, hi) if down else (hi, lo)
                mine = ((self.fwd_out if down else self.bwd_in) if self.topo.rank == lo
                        else (self.fwd_in if down else self.bwd_out))
                if not isinstance(mine, Link):
                    continue                    # a peer-memory link: no communicator behind it
                t = torch.zeros(1, device=self.device)
                if self.topo.rank == src:
                    dist.send(t, dst, group=groups[j])
                else:
                    dist.recv(t, src, group=groups[j])
        if self.cuda:
            torch.cuda.synchronize(self.device)

    # -- context managers --------------------------------------------------------------------------
    def _on_compute(self):
        return torch.cuda.stream(self.compute) if self.cuda else contextlib.nullcontext()

    def _amp(self):
        if self._amp_open:
            return contextlib.nullcontext()
        if self.autocast:
            return torch.autocast(device_type=self.device.type, dtype=torch.bfloat16)
        return contextlib.nullcontext()

    def _prof(self, name: str, op: Op, is_target: bool = False):
        if self.profiler is None:
            return contextlib.nullcontext()
        return self.profiler.operation(name, op.batch, op.view, op.ub, is_target, self.topo.stage)

    # -- feeder side -------------------------------------------------------------------------------
    def start_watchdog(self) -> None:
        from .watchdog import Watchdog
        rt = self.cfg["runtime"]
        if self.topo.world <= 1 or not rt.get("heartbeat_s"):
            return
        self.watchdog = Watchdog(self.topo.store, self.topo.rank, self.topo.world, rt["heartbeat_s"], rt["timeout_s"],
                                 progress=lambda: self.op_count, on_failure=self._peer_failed,
                                 busy=lambda: self._in_op)
        self.watchdog.start()

    def _peer_failed(self, exc: BaseException) -> None:
        if self.error is None:
            self.error = exc
            self.losses.put((-1, exc))

    def start(self) -> None:
        self.start_watchdog()
        self.thread = threading.Thread(target=self._run_guarded, name=f"tspipe-exec-{self.topo.rank}", daemon=True)
        self.thread.start()

    def join(self, timeout: Optional[float] = None) -> None:
        if self.thread is not None:
            self.thread.join(timeout)
        if self.error is not None:
            raise EngineError(f"stage engine on rank {self.topo.rank} failed") from self.error

    def _run_guarded(self) -> None:
        try:
            if self.autocast and self.cuda:
                # One autocast region for the executor's whole life: the bf16 copies of the weights are
                # then cast once per optimizer step (the cache is dropped in _optimize) instead of once per
                # microbatch forward.  Teacher weights take part in the cache only if they are flagged as
                # requiring grad; they are only ever used under no_grad.
                for p in self.target.parameters():
                    p.requires_grad_(True)
                self._amp_ctx = torch.autocast(device_type="cuda", dtype=torch.bfloat16)
                self._amp_ctx.__enter__()
                self._amp_open = True
            self.run()
        except BaseException as e:  # noqa: BLE001 - reported to the owner thread
            first = self.error is None
            if first:
                self.error = e
            Log.e(f"rank {self.topo.rank} executor died:\n{traceback.format_exc()}")
            self.losses.put((-1, e))
            if first:
                try:
                    self.topo.store.set(f"dead/{self.topo.rank}", repr(e).encode()[:2000])
                except Exception:
                    pass
        finally:
            if self.watchdog is not None:
                # an orderly exit says good-bye; after an error the death notice above is what the peers read,
                # and this rank stops beating either way
                if self.error is None:
                    self.watchdog.stop()
                else:
                    self.watchdog.halt()

    # -- availability ------------------------------------------------------------------------------
    def _pump(self, block: bool) -> bool:
        try:
            msg = self.inbox.get(timeout=0.2) if block else self.inbox.get_nowait()
        except queue.Empty:
            return False
        if isinstance(msg, StopMsg):
            self.last_batch = msg.last_batch
            self._flushing = False
        elif isinstance(msg, FlushMsg):
            self.last_batch = msg.last_batch
            self._flushing = True
        elif isinstance(msg, EpochMsg):
            self.force_steps.add(msg.batch_id)
        elif isinstance(msg, FeedMsg):
            self.feeds[msg.batch_id] = msg
            self.highest_fed = max(self.highest_fed, msg.batch_id)
        else:
            raise EngineError(f"unknown message {msg!r}")
        return True

    def _have_batch(self, b: int) -> bool:
        """Block until batch ``b`` has been fed (True) or feeding stopped before it (False)."""
        deadline = time.monotonic() + float(self.cfg["runtime"]["timeout_s"])
        while True:
            if b <= self.highest_fed:
                return True
            if self.last_batch is not None and b > self.last_batch:
                return False
            if self.error is not None:
                raise EngineError("stopping: a peer rank failed") from self.error
            if not self._pump(block=True):
                self._check_peers()
                if time.monotonic() > deadline:
                    raise EngineError(f"rank {self.topo.rank}: no batch {b} and no stop within the timeout")

    def _check_peers(self) -> None:
        if self.on_idle is not None:
            self.on_idle()

    # -- main loop ---------------------------------------------------------------------------------
    def run(self) -> None:
        from . import context
        context.set_current(context.RuntimeContext(self.topo, self.fused,
                                                   bool(self.cfg["runtime"].get("peer_memory", True)) and self.cuda))
        b = 1
        while True:
            if not self._have_batch(b):
                self._drain()
                if not self._flushing:
                    return
                # flushed: resume with batch b as a pipeline-fill batch
                self._flushing = False
                self.last_batch = None
                self.fill_batches.add(b)
                self._fwd_iter, self._fwd_peek = self._fwd_keys(b), None
                if self.on_flushed is not None:
                    self.on_flushed(b - 1)
                continue
            prev_kind = None
            for op in self._block_ops(b):
                if prev_kind == OpKind.B and op.kind != OpKind.B:
                    self._dp_reduce_early()         # this replica's gradients of batch b are complete
                self._dispatch(op)
                prev_kind = op.kind
            self._retire(b)
            b += 1

    def _is_fill(self, b: int) -> bool:
        return b in self.fill_batches

    def _block_ops(self, b: int):
        """Yield the ops of batch block ``b``; resolves 'does batch b+1 exist' lazily, right before
        the first look-ahead teacher forward."""
        spec, j = self.spec, self.topo.stage
        full = batch_block(spec, j, b, None, fill=self._is_fill(b))
        decided: Optional[bool] = None
        for op in full:
            if op.kind == OpKind.T and op.batch == b + 1:
                if decided is None:
                    decided = self._have_batch(b + 1)
                if not decided:
                    continue
            yield op

    def _dispatch(self, op: Op) -> None:
        self.op_count += 1
        self._in_op = True
        try:
            self._dispatch_op(op)
        finally:
            self._in_op = False

    def _dispatch_op(self, op: Op) -> None:
        if op.kind == OpKind.T:
            self._forward(op, teacher=True)
        elif op.kind == OpKind.O:
            self._forward(op, teacher=False)
        elif op.kind == OpKind.B:
            self._backward(op)
        elif op.kind == OpKind.LOSS:
            self._loss(op)
        elif op.kind == OpKind.OPT:
            self._optimize(op)

    # -- input acquisition ---------------------------------------------------------------------------
    def _net(self, teacher: bool) -> str:
        return "t" if teacher else "o"

    def _user_view(self, teacher: bool, view: int) -> int:
        """Which fed view a (net, view) pair consumes.  SSL: schedule view v <-> ``view_{v+1}`` for both
        nets; KD: teacher (view 1) takes ``view_2`` and the student (view 0) ``view_1``
        (`gpu_task.py:548-575`)."""
        return view

    def _stage0_input(self, op: Op, teacher: bool) -> List[Any]:
        msg = self.feeds[op.batch]
        cache = getattr(msg, "_scattered", None)
        if cache is None:
            cache = {}
            msg._scattered = cache
        v = self._user_view(teacher, op.view)
        if v not in cache:
            cache[v] = self.sg.scatter(msg.views[v], self.U)
        ub = cache[v][op.ub]
        data = ub.value if isinstance(ub, Batch) else ub
        if self.cuda:
            # Online and target network read the same views: copy to the device and convert (bf16, channels-last,
            # one kernel) once per view and microbatch, on the compute stream that both forwards run on.
            prepared = getattr(msg, "_prepared", None)
            if prepared is None:
                prepared = {}
                msg._prepared = prepared
            pkey = (v, op.ub)
            if pkey not in prepared:
                if msg.ready_event is not None:
                    torch.cuda.current_stream().wait_event(msg.ready_event)
                data = pt.tree_map_tensors(lambda t: t if t.is_cuda else self._h2d(t), data)
                if self._conv_input():
                    data = pt.tree_map_tensors(_to_conv_input, data)
                prepared[pkey] = data
            data = prepared[pkey]
        return data

    def _can_merge_views(self, rt: Dict[str, Any]) -> bool:
        """Two views, no nano-batch split: both views of a microbatch go through every stage as ONE forward (and
        one backward) over the stacked batch, and cross every stage boundary as one stacked item: the schedule's
        items of view 0 carry both views, its items of view 1 are skipped on every stage.  Every BatchNorm keeps
        per-view statistics (``ops.bn.segments``), so the numbers are those of two separate forwards; the kernels
        are twice as large and half as many, which is what a B200 needs at ~128 samples per view.  Requires that
        all batch-statistics layers are :class:`DeferredBatchNorm` (the only ones that know about stacked views);
        all ranks must agree, so the decision is the minimum over the job."""
        from ..batchnorm import DeferredBatchNorm
        from torch.nn.modules.batchnorm import _BatchNorm
        ok = bool(rt.get("merge_views", True) and not self.kd and self.S == 1
                  and len(self.spec.student_views) == 2 and len(self.spec.teacher_views) == 2)
        if ok:
            for net in (self.online, self.target):
                for m in net.modules():
                    if isinstance(m, _BatchNorm) and not isinstance(m, DeferredBatchNorm):
                        ok = False
        if self.topo.world > 1 and (self.topo.pp > 1):
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(int(flag.item()))
        return ok

    def _conv_input(self) -> bool:
        """True when both networks start with a convolution under bf16 autocast: the cast that autocast would
        do per network and the channels-last conversion can then be one shared kernel per view."""
        flag = getattr(self, "_conv_input_flag", None)
        if flag is None:
            def first_leaf(m):
                while True:
                    ch = list(m.children())
                    if not ch:
                        return m
                    m = ch[0]
            flag = bool(self.autocast and self.channels_last and
                        all(isinstance(first_leaf(m), nn.Conv2d) for m in (self.online, self.target)))
            self._conv_input_flag = flag
        return flag

    def _h2d(self, t: torch.Tensor) -> torch.Tensor:
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(self.copy_stream):
            d = t.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        cur.wait_event(ev)
        d.record_stream(cur)
        return d

    def _recv_forward(self, op: Op, teacher: bool) -> Any:
        """Upstream activation for ``op``: list (per nano-batch for the student, one for the teacher)
        of stage-input pytrees.  Receives are posted in crossing order, ``prefetch`` items ahead."""
        key = (op.kind, op.batch, op.view, op.ub)
        while key not in self.fwd_posted:
            nxt = self._next_fwd_key(blocking=True)
            self._post_forward(nxt)
        depth = int(self.cfg["runtime"].get("prefetch", 2))
        while len(self.fwd_posted) <= depth:
            nxt = self._next_fwd_key(blocking=False)
            if nxt is None:
                break
            self._post_forward(nxt)
        pieces = self.fwd_posted.pop(key)
        return [(_rebuild(h.wait(), others, tree, wrapped), flags) for h, tree, wrapped, others, flags in pieces]

    def _fwd_keys(self, start: int = 1):
        b = start
        while True:
            for o in batch_block(self.spec, self.topo.stage, b, None, fill=self._is_fill(b)):
                if o.kind in (OpKind.T, OpKind.O) and not (self.merge_views and o.view != 0):
                    yield o                 # (stacked views: the item of view 0 carries both, view 1 never crosses)
            b += 1

    def _next_fwd_key(self, blocking: bool) -> Optional[Op]:
        """Next forward item in crossing order.  Non-blocking mode returns None rather than wait for
        an unknown batch or for an unpublished shape announcement."""
        while True:
            if self._fwd_peek is None:
                self._fwd_peek = next(self._fwd_iter)
            o = self._fwd_peek
            if self.last_batch is not None and o.batch > self.last_batch:
                # never fed: it will not cross the link.  Items of batch last+1 are look-ahead teacher
                # forwards interleaved with real items of batch `last`; anything later ends the stream.
                if o.batch > self.last_batch + 1:
                    if blocking:
                        raise EngineError("forward item requested beyond the last fed batch")
                    return None
                self._fwd_peek = None
                continue
            if o.batch > self.highest_fed:
                if not blocking:
                    self._pump(block=False)
                    if o.batch > self.highest_fed:
                        return None
                elif not self._have_batch(o.batch):
                    self._fwd_peek = None
                    continue
            if not blocking:
                if not self.meta.cached(f"f{self.topo.stage - 1}", self._net(o.kind == OpKind.T), o.batch):
                    return None
            self._fwd_peek = None
            return o

    def _post_forward(self, o: Op) -> None:
        net = self._net(o.kind == OpKind.T)
        meta = self.meta.fetch(f"f{self.topo.stage - 1}", net, o.batch)
        self.fwd_posted[(o.kind, o.batch, o.view, o.ub)] = [
            (self.fwd_in.post_recv([(sh, dt) for sh, dt, _ in specs]), tree, wrapped, others,
             [rg for _, _, rg in specs]) for specs, tree, wrapped, others in meta]

    # -- forward -------------------------------------------------------------------------------------
    def _forward(self, op: Op, teacher: bool) -> None:
        first, last = self.topo.is_first, self.topo.is_last
        module = self.target if teacher else self.online
        n_piece = 1 if teacher else self.S
        merged = self.merge_views
        if merged and op.view != 0:
            return                                  # done together with view 0
        with self._on_compute(), self._prof("compute", op, teacher):
            if first and merged:
                both = [self._stage0_input(Op(op.kind, op.batch, v, op.ub), teacher) for v in (0, 1)]
                data = pt.tree_map_tensors_multi(lambda a, b: torch.cat([a, b]), both[0], both[1])
                pieces = [(data, None)]
            elif first:
                data = self._stage0_input(op, teacher)
                pieces = [(d, None) for d in ([data] if n_piece == 1 else pt.generic_scatter(data, n_piece))]
            else:
                pieces = self._recv_forward(op, teacher)
            outs, stored_in, stored_out = [], [], []
            gin_idx: List[int] = []
            gout_idx: List[int] = []
            for x, flags in pieces:
                leaves, tree, wrapped = pt.flatten(x)
                if not teacher and not first:
                    # the sender says which tensor leaves carry a gradient back (same order as the tensors)
                    tensor_pos = [i for i, l in enumerate(leaves) if isinstance(l, torch.Tensor)]
                    gin_idx = [i for i, rg in zip(tensor_pos, flags) if rg]
                    for i in gin_idx:
                        leaves[i] = leaves[i].detach().requires_grad_(True)
                    x = pt.unflatten(leaves, tree, wrapped)
                if self.channels_last:
                    x = pt.tree_map_tensors(_to_channels_last, x)
                slot = None
                with _bn_segments(2 if merged else 1):
                    if teacher:
                        y = self._teacher_forward(module, x)
                        self.bn_group_target.step(2 if merged else 1)
                    else:
                        y = None
                        if self.student_graphs is not None:
                            y, slot = self.student_graphs.forward((op.view, op.ub), x, 2 if merged else 1)
                        if slot is None:
                            with self._amp():
                                y = module(x)
                        self.bn_group_online.step(2 if merged else 1)
                outs.append(y)
                if not teacher:
                    oleaves = pt.flatten(y)[0]
                    gout_idx = [i for i, l in enumerate(oleaves)
                                if isinstance(l, torch.Tensor) and l.requires_grad and l.dim() > 0]
                    stored_in.append(leaves)
                    stored_out.append(oleaves)
            if not teacher:
                self.acts[(op.batch, op.view, op.ub)] = _Stored(stored_in, stored_out, gin_idx, gout_idx, slot)
            if merged and last:
                # the loss sees the two views as two outputs again (halves of the stacked batch)
                for v in (0, 1):
                    half = pt.tree_map_tensors(lambda t, v=v: t.chunk(2)[v] if t.dim() > 0 else t, outs[0])
                    if teacher:
                        self.t_out.setdefault((op.batch, v), [None] * self.U)[op.ub] = half
                    else:
                        self.o_out.setdefault((op.batch, v), [None] * self.U)[op.ub] = [half]
            elif not last:
                self._send_forward(op, teacher, outs)
            else:
                key = (op.batch, op.view)
                if teacher:
                    self.t_out.setdefault(key, [None] * self.U)[op.ub] = outs[0]
                else:
                    self.o_out.setdefault(key, [None] * self.U)[op.ub] = outs

    def _teacher_forward(self, module: nn.Module, x: Any) -> Any:
        """Teacher stage forward (no autograd).  With ``runtime.cuda_graphs`` the whole stage forward of a
        given input shape is captured once into a CUDA graph and replayed afterwards: one launch per
        microbatch instead of several hundred (weights are re-cast inside the graph, BatchNorm statistics
        accumulate on the device; only the commit counter lives on the host)."""
        use_graph = (self.cuda and self.cfg["runtime"].get("cuda_graphs", False)
                     and not any(isinstance(m, nn.Dropout) and m.p > 0 and m.training for m in module.modules()))
        if not use_graph:
            with torch.no_grad(), self._amp():
                return module(x)
        # stage inputs / outputs may be pytrees (dicts of tensors in the BERT stages): the graph is keyed by the
        # tensor leaves' geometry and the values of the other leaves, and works on static copies of the tensors
        leaves, tree, wrapped = pt.flatten(x)
        tpos = [i for i, l in enumerate(leaves) if isinstance(l, torch.Tensor)]
        if not tpos or any(not leaves[i].is_cuda for i in tpos):
            with torch.no_grad(), self._amp():
                return module(x)
        key = (str(tree), wrapped, tuple((tuple(leaves[i].shape), leaves[i].dtype, leaves[i].stride()) for i in tpos),
               tuple(repr(l) for i, l in enumerate(leaves) if i not in tpos))
        entry = self._teacher_graphs.get(key)
        if entry is None or entry[0] < 2:           # two eager calls first (library autotuning, lazy inits)
            self._teacher_graphs[key] = (0 if entry is None else entry[0] + 1, None, None, None)
            with torch.no_grad(), self._amp():
                return module(x)
        if entry[1] is None:
            static_leaves = [l.clone() if isinstance(l, torch.Tensor) else l for l in leaves]
            static_in = pt.unflatten(static_leaves, tree, wrapped)
            graph = torch.cuda.CUDAGraph()
            from .stage_graph import capture

            def body():
                with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.autocast,
                                                     cache_enabled=False):
                    return module(static_in)
            from ..ops import fused as _fused
            n0 = _fused.LAUNCHES
            static_out = capture(graph, self._graph_stream, None, body)
            self._teacher_graph_launches[key] = _fused.LAUNCHES - n0
            _fused.LAUNCHES = n0
            entry = (2, graph, static_leaves, static_out)
            self._teacher_graphs[key] = entry
            # the capture itself did not execute anything: fall through to a replay
        _, graph, static_leaves, static_out = entry
        for i in tpos:
            static_leaves[i].copy_(leaves[i])
        graph.replay()
        from ..ops import fused as _fused
        _fused._count(self._teacher_graph_launches.get(key, 0))
        return pt.tree_map_tensors(lambda t: t.clone(), static_out)

    def _send_forward(self, op: Op, teacher: bool, outs: List[Any]) -> None:
        net = self._net(teacher)
        meta, tensors = [], []
        for y in outs:
            leaves, tree, wrapped = pt.flatten(y)
            ts = [l.detach() for l in leaves if isinstance(l, torch.Tensor)]
            others = [(i, l) for i, l in enumerate(leaves) if not isinstance(l, torch.Tensor)]
            rgs = [bool(l.requires_grad and l.dim() > 0) for l in leaves if isinstance(l, torch.Tensor)]
            meta.append(([(tuple(t.shape), t.dtype, rg) for t, rg in zip(ts, rgs)], tree, wrapped, others))
            tensors.append(ts)
        self.meta.publish(f"f{self.topo.stage}", net, op.batch, meta)
        for ts in tensors:
            self.fwd_out.send(ts)

    # -- loss ----------------------------------------------------------------------------------------
    def _loss(self, op: Op) -> None:
        b = op.batch
        msg = self.feeds[b]
        with self._on_compute(), self._prof("loss", op):
            online_full, leaf_sets = [], []
            for v in self.spec.student_views:
                nano_outs = [y for ub in self.o_out.pop((b, v)) for y in ub]          # U*S stage outputs
                flat = [pt.flatten(y) for y in nano_outs]
                tree, wrapped = flat[0][1], flat[0][2]
                cat_leaves = []
                for i, l in enumerate(flat[0][0]):
                    if isinstance(l, torch.Tensor) and l.dim() > 0:
                        t = torch.cat([f[0][i].detach() for f in flat]) if len(flat) > 1 else l.detach()
                        if l.requires_grad:
                            t.requires_grad_(True)
                        cat_leaves.append(t)
                    else:
                        cat_leaves.append(l.detach() if isinstance(l, torch.Tensor) else l)
                leaf_sets.append((v, cat_leaves, [f[0] for f in flat]))
                online_full.append(pt.unwrap(pt.unflatten(cat_leaves, tree, wrapped)))
            target_full = []
            for v in self.spec.teacher_views:
                outs = self.t_out.pop((b, v))
                target_full.append(pt.unwrap(self.sg.gather([Batch(pt.unwrap(o)) for o in outs])))
            with self._amp():
                if self.kd:
                    labels = msg.labels
                    if self.cuda and labels is not None:
                        labels = pt.tree_map_tensors(lambda t: t if t.is_cuda else self._h2d(t), labels)
                    loss = self.loss_fn(online_full[0], target_full[0], labels, self.args, self.extra_args, msg.epoch)
                else:
                    loss = self.loss_fn(online_full[0], online_full[1], target_full[0], target_full[1],
                                        self.args, self.extra_args)
            self._report_loss(b, loss.detach())
            torch.autograd.backward(loss)
            n_nano = self.U * self.S
            for v, cat_leaves, per_nano in leaf_sets:
                grads_per_nano: List[List[torch.Tensor]] = [[] for _ in range(n_nano)]
                for i, t in enumerate(cat_leaves):
                    if isinstance(t, torch.Tensor) and t.requires_grad:
                        g = t.grad if t.grad is not None else torch.zeros_like(t)
                        sizes = [leaves[i].shape[0] for leaves in per_nano]
                        for k, gk in enumerate(g.split(sizes)):
                            grads_per_nano[k].append(gk)
                for k in range(n_nano):
                    self.out_grads[(b, v, k)] = grads_per_nano[k]

    def _report_loss(self, b: int, loss: torch.Tensor) -> None:
        if self.cuda:
            host = torch.empty((), dtype=torch.float32, pin_memory=True)
            host.copy_(loss.float(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.losses.put((b, (host, ev)))
        else:
            self.losses.put((b, float(loss)))

    # -- backward ------------------------------------------------------------------------------------
    def _backward(self, op: Op) -> None:
        b, v, k = op.batch, op.view, op.ub
        ub, piece = divmod(k, self.S)
        if self.merge_views and v != 0:
            return                                  # done together with view 0
        st = self.acts[(b, v, ub)]
        with self._on_compute(), self._prof("backward", op):
            outs = [st.outputs[piece][i] for i in st.grad_out_idx]
            if self.merge_views and self.topo.is_last:
                g0, g1 = self.out_grads.pop((b, 0, k)), self.out_grads.pop((b, 1, k))
                grads = [torch.cat([a, c]) for a, c in zip(g0, g1)]
            elif self.topo.is_last:
                grads = self.out_grads.pop((b, v, k))
            else:
                grads = self._recv_backward(op)
            if st.graph is not None:
                gin = self.student_graphs.backward(st.graph, grads)
                if not self.topo.is_first:
                    self.bwd_out.send(gin)
            else:
                if outs:
                    torch.autograd.backward(outs, grads)
                if not self.topo.is_first:
                    gin = []
                    for i in st.grad_in_idx:
                        leaf = st.inputs[piece][i]
                        gin.append(leaf.grad if leaf.grad is not None else torch.zeros_like(leaf))
                    self.bwd_out.send(gin)
            st.outputs[piece] = None
            st.inputs[piece] = None
            if all(o is None for o in st.outputs):
                del self.acts[(b, v, ub)]

    def _recv_backward(self, op: Op) -> List[torch.Tensor]:
        """Gradient of one nano-batch from downstream; receives for the next ``prefetch`` backward items
        of the batch are posted too (their shapes are those of the stored stage outputs)."""
        order = self._bwd_order.get(op.batch)
        if order is None:
            order = [o for o in self.spec.backward_items(op.batch, self.topo.stage)
                     if not (self.merge_views and o.view != 0)]
            self._bwd_order = {op.batch: order}
        i = next(n for n, o in enumerate(order) if o.view == op.view and o.ub == op.ub)
        depth = int(self.cfg["runtime"].get("prefetch", 2))
        for o in order[i: i + 1 + depth]:
            key = (o.batch, o.view, o.ub)
            if key in self.bwd_posted:
                continue
            ub, piece = divmod(o.ub, self.S)
            st = self.acts[(o.batch, o.view, ub)]
            specs = [(tuple(st.outputs[piece][n].shape), st.outputs[piece][n].dtype) for n in st.grad_out_idx]
            self.bwd_posted[key] = self.bwd_in.post_recv(specs)
        return self.bwd_posted.pop((op.batch, op.view, op.ub)).wait()

    # -- optimize ------------------------------------------------------------------------------------
    def _optimize(self, op: Op) -> None:
        b = op.batch
        msg = self.feeds[b]
        if msg.new_momentum is not None:
            self.momentum = msg.new_momentum
        if msg.new_lr is not None and self.optimizer is not None:
            lrs = msg.new_lr if isinstance(msg.new_lr, (list, tuple)) else [msg.new_lr] * len(self.optimizer.param_groups)
            for g, lr in zip(self.optimizer.param_groups, lrs):
                g["lr"] = lr
        if self.ga > 1:
            self._have_batch(b + 1)        # an epoch-boundary notice for b precedes the next feed / stop
        force = msg.force_step or b in self.force_steps
        skip = self.skip_optimizer or ((self.ga_count + 1) % self.ga != 0 and not force)
        with self._on_compute(), self._prof("optimize", op):
            if skip:
                if self.ga > 1 and not self.skip_optimizer:
                    self.ga_count += 1
                else:
                    self.flat_online.zero_grad()
                return
            self.flat_online.collect_stray_grads()
            if self.ga > 1:
                self.flat_online.grad.div_(self.ga_count + 1)
                self.ga_count = 0
            self._dp_sync()
            if self._dp_event is not None:          # the early half of the data-parallel step ran on the side stream
                torch.cuda.current_stream().wait_event(self._dp_event)
                self._dp_event = None
            if hasattr(self.updater, "before_step"):
                self.updater.before_step(self.momentum)
            if self.optimizer is not None:
                self.optimizer.step()
            self.updater.step(self.momentum)
            if self.async_emu:
                # `async_param_update_emulation` (`tspipe/gpu_task.py:58-66,351-356`): the student of batch b
                # runs on version b-2 as well, i.e. two interleaved parameter trajectories.  The live buffer now
                # holds version b; park it and bring back version b-1 for the next batch.
                if self._alt_params is None:
                    self._alt_params = self._initial_params
                    self._initial_params = None
                tmp = self.flat_online.data.clone()
                self.flat_online.data.copy_(self._alt_params)
                self._alt_params = tmp
            self.flat_online.zero_grad()
            if self._amp_open:
                torch.clear_autocast_cache()
            if self.cuda:
                from ..ops import conv as _conv
                from ..ops import gemm as _gemm
                _conv.clear_weight_cache()          # bf16 weight copies of the tcgen05 convolutions ...
                _gemm.clear_weight_cache()          # ... and linear layers
            self.steps_done += 1

    def _dp_reduce_early(self) -> None:
        """Start the data-parallel gradient reduction as soon as the last backward item of the batch has been
        enqueued, on the side stream: the schedule places the look-ahead teacher forwards of the next batch between
        the backward wave and the optimizer step, so the peer reads (and the wait for the slowest replica) run
        behind that forward instead of in front of the step.  DDP in the reference's baselines overlaps its
        all-reduce buckets with backward (`benchmarks/moco-v3/main.py:249-254`); the pipelined runtime has none."""
        opt = self.optimizer
        if not (self.dp_fused and self.cuda and self.ga == 1 and not self.skip_optimizer
                and hasattr(opt, "dp_reduce") and self._dp_event is None
                and self.cfg["runtime"].get("dp_early_reduce", True)):
            return
        with self._on_compute():
            self.flat_online.collect_stray_grads()
            ready = torch.cuda.Event()
            ready.record()
        with torch.cuda.stream(self.dp_stream):
            self.dp_stream.wait_event(ready)
            opt.dp_reduce()
            self._dp_event = torch.cuda.Event()
            self._dp_event.record()

    def _dp_sync(self) -> None:
        if self.topo.dp_group is None:
            return
        opt = self.optimizer
        if opt is not None and getattr(opt, "handles_dp", False):
            return          # the fused reduce-scatter + step path does its own synchronisation
        dist.all_reduce(self.flat_online.grad, op=dist.ReduceOp.SUM, group=self.topo.dp_group)
        self.flat_online.grad.div_(self.topo.dp)

    # -- retire / drain ------------------------------------------------------------------------------
    def _retire(self, b: int) -> None:
        self.feeds.pop(b - 1, None)
        for link in (self.fwd_in, self.fwd_out, self.bwd_in, self.bwd_out):
            if link is not None and hasattr(link, "poll"):
                link.poll()                 # a device-side wait of a peer link that gave up surfaces here
        if self.on_batch_done is not None:
            self.on_batch_done(b)

    def _drain(self) -> None:
        for link in (self.fwd_out, self.bwd_out):
            if link is not None:
                link.flush()
        if self.cuda:
            self.compute.synchronize()
        for link in (self.fwd_in, self.bwd_in):
            if link is not None and hasattr(link, "poll"):
                link.poll(sync=True)


def _bn_segments(n: int):
    from ..ops import bn as _bn
    return _bn.segments(n)


def _to_conv_input(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 4 and t.dtype in (torch.float32, torch.bfloat16):
        return t.to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    return t


def _to_channels_last(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous(memory_format=torch.channels_last) if t.dim() == 4 else t


def _rebuild(tensors: List[torch.Tensor], others: List[Tuple[int, Any]], tree: Any, wrapped: bool) -> Any:
    n = len(tensors) + len(others)
    leaves: List[Any] = [None] * n
    taken = set()
    for i, l in others:
        leaves[i] = l
        taken.add(i)
    it = iter(tensors)
    for i in range(n):
        if i not in taken:
            leaves[i] = next(it)
    return pt.unflatten(leaves, tree, wrapped)
