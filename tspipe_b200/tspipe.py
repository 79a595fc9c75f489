"""User-facing facade: :class:`TSPipe`.

Same constructor, callbacks and methods as the reference facade (`tspipe/tspipe.py:51-64`
ctor, `:394-445` ``feed``, `:447` ``feed_epoch``, `:452-484` ``stop``, `:511-519`
``update_momentum`` / ``update_lr``, `:237` ``is_primary``, `:521-583` ``split_module``), over
a different runtime:

* **launch** - two ways.  *Launcher mode*: the script itself runs once per device under
  ``torchrun`` (``RANK`` / ``WORLD_SIZE`` in the environment); every rank constructs
  ``TSPipe`` with the same arguments and calls ``feed`` / ``stop`` in lockstep, the way
  data-parallel scripts do.  *Spawn mode* (the reference's way, `tspipe/tspipe.py:118-127`):
  one user process constructs ``TSPipe`` with ``--tspipe-config --ip --rank --num-nodes``; it
  spawns one worker process per local device and feeds them through shared-memory queues.
* **no scheduler rank, no per-task RPC** - each worker derives its own column of the
  schedule (:mod:`tspipe_b200.schedule`); the only cross-process control traffic is "batch
  ``b`` is fed", lr / momentum updates, epoch boundaries, stop, and loss scalars.
* ranks form a ``dp x pp`` grid (``runtime.dp_replicas``); the reference supports ``dp = 1``.
"""
from __future__ import annotations

import os
import queue
import time
import warnings
from argparse import Namespace
from collections import OrderedDict
from enum import Enum
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn

from .batch_ops import Batch, BatchQueue, ScatterGatherFn, defaultScatterGatherFn
from .batchnorm import DeferredBatchNorm
from .config import load_yaml, merge_config, parse_cli
from .logger import Log
from .utils import pytree as pt

__all__ = ["TSPipe", "TSPipeMode", "BalanceError"]


class TSPipeMode(Enum):
    SELF_SUPERVISED_MOMENTUM = 1
    SUPERVISED_MOMENTUM = 2


class BalanceError(ValueError):
    pass


def verify_module(module: nn.Sequential) -> None:
    """`tspipe/utils.py:48-67`: a cut-able model is an ``nn.Sequential`` without duplicate children."""
    if not isinstance(module, nn.Sequential):
        raise TypeError("module must be nn.Sequential to be partitioned")
    if len(list(module.named_children())) != len(module):       # named_children() drops repeated modules
        raise ValueError("module with duplicate children is not supported")


def split_sequential(children: Iterable[Tuple[str, nn.Module]], balance: Sequence[int]) -> List[nn.Sequential]:
    parts: List[nn.Sequential] = []
    layers: "OrderedDict[str, nn.Module]" = OrderedDict()
    j = 0
    for name, layer in children:
        if name in layers:
            name = f"{name}_"
        layers[name] = layer
        if len(layers) == balance[j]:
            parts.append(nn.Sequential(layers))
            layers = OrderedDict()
            j += 1
    return parts


def split_module(module_online: nn.Sequential, module_target: nn.Sequential,
                 module_predictor: Optional[nn.Sequential], balance_online: Sequence[int],
                 balance_target: Sequence[int]) -> Tuple[List[nn.Sequential], List[nn.Sequential]]:
    """Cut ``online ++ predictor`` and ``target`` by child counts (`tspipe/tspipe.py:521-583`).
    Children of the predictor whose names collide with the online net's get a ``predictor_`` prefix
    (the reference silently overwrites them)."""
    balance_online, balance_target = list(balance_online), list(balance_target)
    n_on = len(module_online) + (len(module_predictor) if module_predictor is not None else 0)
    if n_on != sum(balance_online):
        raise BalanceError("online module and sum of balance have different length "
                           f"(module: {n_on}, sum of balance: {sum(balance_online)})")
    if len(module_target) != sum(balance_target):
        raise BalanceError("target module and sum of balance have different length "
                           f"(module: {len(module_target)}, sum of balance: {sum(balance_target)})")
    for bal in (balance_online, balance_target):
        if any(x <= 0 for x in bal):
            raise BalanceError(f"all balance numbers must be positive integer (balance: {bal})")
    online_children = list(module_online.named_children())
    if module_predictor is not None:
        taken = {n for n, _ in online_children}
        for n, m in module_predictor.named_children():
            online_children.append((f"predictor_{n}" if n in taken else n, m))
    return (split_sequential(online_children, balance_online),
            split_sequential(module_target.named_children(), balance_target))


def default_balance(n_children: int, n_parts: int) -> List[int]:
    base, rem = divmod(n_children, n_parts)
    if base == 0:
        raise BalanceError(f"cannot cut {n_children} children into {n_parts} partitions")
    return [base + (1 if i < rem else 0) for i in range(n_parts)]


def rebind_optimizer(optimizer: torch.optim.Optimizer, local_params: Sequence[nn.Parameter]) -> None:
    """Keep only the parameters of this rank's partition in each param group
    (`tspipe/tspipe.py:169-180`, `tspipe/gpu_worker.py:456-461`)."""
    local = {id(p) for p in local_params}
    for g in optimizer.param_groups:
        g["params"] = [p for p in g["params"] if id(p) in local]
    for p in list(optimizer.state.keys()):
        if id(p) not in local:
            del optimizer.state[p]


class TSPipe:
    def __init__(self,
                 module_online: nn.Sequential,
                 module_target: nn.Sequential,
                 module_predictor: Optional[nn.Sequential],
                 optimizer: torch.optim.Optimizer,
                 loss_fn: Callable,
                 target_update_fn: Optional[Callable],
                 momentum: float,
                 artifact_dir: str = "",
                 tspipe_mode: TSPipeMode = TSPipeMode.SELF_SUPERVISED_MOMENTUM,
                 target_train_mode: bool = True,
                 extra_args: Namespace = Namespace(),
                 scatter_gather_fn: ScatterGatherFn = defaultScatterGatherFn,
                 config: Optional[Dict[str, Any]] = None,
                 argv: Optional[Sequence[str]] = None,
                 device: Optional[Union[str, torch.device]] = None,
                 profiler=None):
        launcher = "RANK" in os.environ and "WORLD_SIZE" in os.environ or dist.is_initialized()
        if config is None:
            self.args = parse_cli(argv, required=not launcher)
            self.config = load_yaml(self.args.tspipe_config)
        else:
            self.args = parse_cli(argv, required=False)
            self.config = merge_config(config)
        self.config["__artifact_dir"] = artifact_dir
        self.module_online, self.module_target, self.module_predictor = module_online, module_target, module_predictor
        self.optimizer, self.loss_fn, self.target_update_fn = optimizer, loss_fn, target_update_fn
        self.momentum = momentum
        self.artifact_dir = artifact_dir
        self.tspipe_mode = tspipe_mode
        self.target_train_mode = target_train_mode
        self.extra_args = extra_args
        self.scatter_gather_fn = scatter_gather_fn
        self.profiler = profiler
        if target_update_fn is None:
            warnings.warn("Target update function is not designated. Target network will not be updated.")

        verify_module(module_online)
        verify_module(module_target)
        if module_predictor is not None:
            verify_module(module_predictor)

        self.batch_q = BatchQueue()
        self.scheduled_lr_update: Dict[int, Any] = {}
        self.scheduled_momentum_update: Dict[int, float] = {}
        self.epoch = 0
        self._epoch_forced: set = set()
        self.last_batch_idx = 0
        self._losses_returned = 0
        self._stopped = False
        from .run_log import ThroughputMeter
        self.meter = ThroughputMeter()          # samples per second as seen by feed()
        self._feed_stream = None
        self._resumed_batch = 0         # batch id of the checkpoint this run resumed from (0 = fresh run)

        if launcher:
            self._init_launcher(device)
        else:
            self._init_spawn(device)

    # ------------------------------------------------------------------------------------------
    # launcher mode
    # ------------------------------------------------------------------------------------------
    def _resolve_grid(self, world: int) -> Tuple[int, int]:
        split = self.config["model_split"]
        rt = self.config["runtime"]
        if split["online"] is not None:
            pp = len(split["online"])
            if split["target"] is None or len(split["target"]) != pp:
                raise BalanceError("model_split.online and model_split.target need one entry per stage each")
        else:
            dp = rt["dp_replicas"] or 1
            pp = world // dp
        dp = rt["dp_replicas"] or world // pp
        if dp * pp != world:
            raise ValueError("The number of devices must equal partitions x dp_replicas "
                             f"(world {world}, partitions {pp}, dp_replicas {dp}).")
        return pp, dp

    def _init_launcher(self, device) -> None:
        from .comm.topology import build_topology, init_distributed
        from .runtime.engine import StageEngine
        rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
        if device is None:
            use_cuda = torch.cuda.is_available() and self.config["runtime"]["backend"] != "gloo"
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
        device = torch.device(device)
        backend = self.config["runtime"]["backend"]
        if backend == "auto":
            backend = "nccl" if device.type == "cuda" else "gloo"
        init_distributed(rank, world, backend, os.environ.get("MASTER_ADDR", "127.0.0.1"),
                         int(os.environ.get("MASTER_PORT", 29500)), device, self.config["runtime"]["timeout_s"])
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", self.world))
        if local_world < self.world and self.config["runtime"]["peer_memory"]:
            # ranks span several nodes: peer-mapped buffers only exist inside a node, use the collectives
            Log.i("multi-node job: peer-memory paths disabled, NCCL collectives are used instead")
            self.config["runtime"]["peer_memory"] = False
        if self.config["runtime"]["placement"] == "split":
            return self._init_split(device)
        pp, dp = self._resolve_grid(self.world)
        self.topo = build_topology(pp, dp, device, timeout_s=self.config["runtime"]["timeout_s"])
        self._build_partitions(pp)
        j = self.topo.stage
        part_on, part_tg = self.partitions_online[j], self.partitions_target[j]
        rebind_optimizer(self.optimizer, list(part_on.parameters()))
        self.engine = StageEngine(self.topo, self.config, part_on, part_tg, self.optimizer, self.loss_fn,
                                  self.target_update_fn, self.momentum,
                                  kd_mode=self.tspipe_mode == TSPipeMode.SUPERVISED_MOMENTUM,
                                  target_train_mode=self.target_train_mode, scatter_gather_fn=self.scatter_gather_fn,
                                  args=self.args, extra_args=self.extra_args, profiler=self.profiler,
                                  ema_plan=self.ema_plans[j] if self.ema_plans else None)
        for i in range(pp):     # the other stages live on other ranks
            if i != j:
                self.partitions_online[i] = None
                self.partitions_target[i] = None
        self._maybe_resume()
        self.engine.on_batch_done = self._on_batch_done
        self._done_batches = 0
        self.num_ubatches = self.engine.U
        self.num_bwd_ubatches = self.engine.U * self.engine.S
        self.mode = "launcher"
        self.engine.start()

    def _init_split(self, device) -> None:
        """Teacher stages on the first ranks of each replica, student stages on the rest."""
        from .runtime.split_engine import SplitKDEngine, SplitTopology
        ssl = self.tspipe_mode != TSPipeMode.SUPERVISED_MOMENTUM
        fn = self.target_update_fn
        if fn is not None and not getattr(fn, "is_ema", False):
            raise ValueError("runtime.placement: split updates the teacher with the momentum rule "
                             "(tspipe_b200.losses.ema_update) or not at all")
        if ssl and fn is None:
            warnings.warn("self-supervised split placement without a target update function: frozen teacher")
        if fn is not None and self.config["runtime"].get("resume"):
            raise ValueError("resuming a momentum teacher in split placement is not supported")
        split = self.config["model_split"]
        if split["online"] is None or split["target"] is None:
            raise BalanceError("split placement needs model_split.online and model_split.target")
        pt_, ps = len(split["target"]), len(split["online"])
        dp = self.config["runtime"]["dp_replicas"] or self.world // (pt_ + ps)
        self.topo = SplitTopology(pt_, ps, dp, device, timeout_s=self.config["runtime"]["timeout_s"],
                                  ema_pairs=fn is not None)
        if self.config["runtime"]["num_ubatch"] is None:
            self.config["runtime"]["num_ubatch"] = max(ps - 1, 1)
        self.config["train"]["deferred_batch_norm"] = False
        n_on = len(self.module_online) + (len(self.module_predictor) if self.module_predictor is not None else 0)
        self.partitions_online, self.partitions_target = split_module(
            self.module_online, self.module_target, self.module_predictor, split["online"], split["target"])
        self.ema_plans = None
        routes = None
        if fn is not None:
            from .runtime.ema_plan import build_ema_plans, split_placement_routes
            routes = split_placement_routes(build_ema_plans(self.partitions_online, self.partitions_target), pt_, ps)
        t = self.topo
        part = self.partitions_target[t.stage] if t.is_teacher else self.partitions_online[t.stage]
        opt = None
        if not t.is_teacher:
            rebind_optimizer(self.optimizer, list(part.parameters()))
            opt = self.optimizer
        self.engine = SplitKDEngine(t, self.config, part, opt, self.loss_fn, self.target_train_mode,
                                    self.scatter_gather_fn, self.args, self.extra_args, ssl=ssl,
                                    momentum=self.momentum, ema_routes=routes)
        self._maybe_resume()
        self.engine.on_batch_done = self._on_batch_done
        self._done_batches = 0
        self.num_ubatches = self.num_bwd_ubatches = self.engine.U
        self.mode = "launcher"
        self.engine.start()

    def _is_loss_rank(self) -> bool:
        t = self.topo
        return bool(getattr(t, "is_loss_rank", t.is_last))

    def _build_partitions(self, pp: int) -> None:
        cfg = self.config
        rt, gp = cfg["runtime"], cfg["gpipe_emulation"]
        n_ub = gp["num_ubatch"] if gp["enabled"] else (rt["num_ubatch"] or max(pp - 1, 1))
        split_s = 1 if gp["enabled"] else rt["bwd_split"]
        if cfg["train"]["deferred_batch_norm"]:
            views_t = 1
            self.module_online = DeferredBatchNorm.convert_deferred_batch_norm(self.module_online, n_ub * split_s)
            self.module_target = DeferredBatchNorm.convert_deferred_batch_norm(self.module_target, n_ub * views_t)
            if self.module_predictor is not None:
                self.module_predictor = DeferredBatchNorm.convert_deferred_batch_norm(self.module_predictor,
                                                                                       n_ub * split_s)
        split = cfg["model_split"]
        n_on = len(self.module_online) + (len(self.module_predictor) if self.module_predictor is not None else 0)
        bal_on = split["online"] or default_balance(n_on, pp)
        bal_tg = split["target"] or default_balance(len(self.module_target), pp)
        self.partitions_online, self.partitions_target = split_module(
            self.module_online, self.module_target, self.module_predictor, bal_on, bal_tg)
        from .skip import Skippable, verify_skippables, wrap_partitions
        for parts in (self.partitions_online, self.partitions_target):
            if any(isinstance(m, Skippable) for p_ in parts for m in p_.children()):
                verify_skippables(nn.Sequential(*[m for p_ in parts for m in p_.children()]))
        self.partitions_online = wrap_partitions(self.partitions_online)
        self.partitions_target = wrap_partitions(self.partitions_target)
        self.ema_plans = None
        if getattr(self.target_update_fn, "is_ema", False):
            from .runtime.ema_plan import build_ema_plans
            self.ema_plans = build_ema_plans(self.partitions_online, self.partitions_target)

    def _on_batch_done(self, b: int) -> None:
        self._done_batches = b
        every = int(self.config["train"]["save_model_every_iter"] or 0)
        # Batch ids restart at 1 in a resumed run (the schedule's warm-up phase runs again); checkpoint names and
        # the batch id stored in them continue from the checkpoint the run started from, so files of the earlier
        # run are never overwritten and the newest file is always the latest state.
        gb = b + self._resumed_batch
        if every > 0 and gb % every == 0 and self.artifact_dir:
            from .ckpt import save_partition
            save_partition(self.artifact_dir, gb, self._partition_id(), self.engine, replica=self.topo.replica)

    def _partition_id(self) -> int:
        """Index of this rank's partition in checkpoint file names: the stage, or in split placement the rank's
        position inside its replica (teacher stages first, then student stages)."""
        return int(getattr(self.topo, "local", self.topo.stage))

    def _maybe_resume(self) -> None:
        path = self.config["runtime"]["resume"]
        if path:
            from .ckpt import load_partition
            self._resumed_batch = load_partition(path, self._partition_id(), self.engine)

    # ------------------------------------------------------------------------------------------
    # spawn mode
    # ------------------------------------------------------------------------------------------
    def _init_spawn(self, device) -> None:
        from .runtime.worker import SpawnedPipeline
        self.mode = "spawn"
        self.rank = self.args.rank
        pp_total = None
        split = self.config["model_split"]
        if split["online"] is not None:
            pp_total = len(split["online"])
        self.pipeline = SpawnedPipeline(self, device, pp_total)
        self.num_ubatches = self.pipeline.n_ubatch
        self.num_bwd_ubatches = self.pipeline.n_ubatch * self.pipeline.bwd_split
        if self.rank != 0:
            self.pipeline.join()

    # ------------------------------------------------------------------------------------------
    # public API
    # ------------------------------------------------------------------------------------------
    def is_primary(self) -> bool:
        return self.rank == 0

    def update_momentum(self, new_momentum: float) -> None:
        self.scheduled_momentum_update[self.batch_q.next_id] = new_momentum

    def update_lr(self, new_lr: Union[float, List[float]]) -> None:
        self.scheduled_lr_update[self.batch_q.next_id] = new_lr

    def feed_epoch(self) -> None:
        """Epoch boundary: the optimizer steps at the last fed batch even if gradient accumulation
        is incomplete (`tspipe/tspipe.py:447-450`, `gpu_task.py:363-365`)."""
        from .runtime.engine import EpochMsg
        self.batch_q.report_epoch_boundary()
        self.epoch += 1
        if self.last_batch_idx > 0:
            if self.mode == "spawn":
                self.pipeline.broadcast(EpochMsg(self.last_batch_idx))
            else:
                self.engine.inbox.put(EpochMsg(self.last_batch_idx))

    def feed(self, view_1: Any, view_2: Any, view_target: Any = None) -> Optional[float]:
        """Feed one mini-batch.  Returns the loss of an *earlier* batch (``None`` during the first
        iterations): the pipeline runs ``runtime.max_inflight`` batches behind the feeder."""
        assert not self._stopped, "pipeline already stopped"
        kd = self.tspipe_mode == TSPipeMode.SUPERVISED_MOMENTUM
        if kd:
            assert view_target is not None, "Supervised learning requires labels."
        else:
            assert view_target is None, "Self-supervised learning does not support labels."
        sg = self.scatter_gather_fn
        ga = int(self.config["optimizer"]["gradient_accumulation"])
        if view_1 is None:
            # launcher mode: a rank that holds neither stage 0 nor the loss stage has nothing to feed
            assert self.mode == "launcher" and not self.topo.is_first and ga == 1, \
                "views may be omitted only on ranks that do not hold stage 0 (and without gradient accumulation)"
            bs = 0
        else:
            bs = sg.batch_size(view_1)
            assert bs == sg.batch_size(view_2)
        if ga > 1 and bs >= 4 * self.num_ubatches * ga:
            minis_1 = [b.value for b in sg.scatter(view_1, ga)]
            minis_2 = [b.value for b in sg.scatter(view_2, ga)]
            minis_t = [b.value for b in sg.scatter(view_target, ga)] if kd else [None] * ga
        else:
            minis_1, minis_2, minis_t = [view_1], [view_2], [view_target]
        loss = None
        self.meter.add(bs)
        for v1, v2, vt in zip(minis_1, minis_2, minis_t):
            bid = self.batch_q.get_new_batch_id()
            self.last_batch_idx = bid
            self._submit(bid, [v1, v2], vt)
            loss = self.wait_forward()
        return loss

    def _submit(self, bid: int, views: List[Any], labels: Any) -> None:
        from .runtime.engine import FeedMsg
        msg = FeedMsg(batch_id=bid,
                      new_lr=self.scheduled_lr_update.pop(bid, None),
                      new_momentum=self.scheduled_momentum_update.pop(bid, None), epoch=self.epoch)
        if self.mode == "spawn":
            self.pipeline.submit(msg, views, labels)
            return
        topo = self.topo
        if topo.is_first:
            msg.views = views
            if topo.is_cuda:
                msg.views, msg.ready_event = self._stage_inputs(views)
        if self._is_loss_rank():
            msg.labels = labels
        max_inflight = int(self.config["runtime"]["max_inflight"])
        while bid - self._done_batches > max_inflight:
            self._raise_if_failed()
            time.sleep(0.0005)
        self._raise_if_failed()
        self.engine.inbox.put(msg)

    def _raise_if_failed(self) -> None:
        err = self.engine.error
        if err is not None:
            from .runtime.engine import EngineError
            raise EngineError(f"pipeline failed on or near rank {self.rank}: {err}") from err

    def _stage_inputs(self, views: List[Any]):
        """Start the host-to-device copies of a whole mini-batch on the feeder's own stream; the
        executor waits on the event, not the host."""
        dev = self.topo.device
        if self._feed_stream is None:
            self._feed_stream = torch.cuda.Stream(dev)
        need = any(t.device.type != "cuda" for v in views for t in pt.tensors_of(v))
        if not need:
            return views, None
        with torch.cuda.stream(self._feed_stream):
            out = [pt.tree_map_tensors(lambda t: t.to(dev, non_blocking=True), v) for v in views]
            ev = torch.cuda.Event()
            ev.record()
        return out, ev

    def wait_forward(self) -> Optional[float]:
        """Loss of the oldest unreported batch if it is ready; blocks only once the feeder is
        ``max_inflight`` batches ahead of the last reported loss (`tspipe/tspipe.py:486-509`)."""
        if self.mode == "spawn":
            return self.pipeline.poll_loss(self.last_batch_idx, int(self.config["runtime"]["max_inflight"]))
        lag = self.last_batch_idx - self._losses_returned
        block = lag >= int(self.config["runtime"]["max_inflight"])
        if self._is_loss_rank():
            return self._pop_loss(block)
        if self.rank == 0:
            return self._remote_loss(block)
        return None

    def _loss_publisher(self) -> bool:
        """The loss stage of replica 0 forwards every loss to rank 0 (the primary) through the store when
        rank 0 does not hold the loss stage itself."""
        t = self.topo
        return self._is_loss_rank() and t.replica == 0 and t.rank != 0

    def _remote_loss(self, block: bool) -> Optional[float]:
        import pickle
        key = f"loss/{self._losses_returned + 1}"
        store = self.topo.store
        deadline = time.monotonic() + float(self.config["runtime"]["timeout_s"])
        while not store.check([key]):
            if not block:
                return None
            self._raise_if_failed()
            if time.monotonic() > deadline:
                raise TimeoutError("no loss within runtime.timeout_s")
            time.sleep(0.001)
        val = pickle.loads(store.get(key))
        try:
            store.delete_key(key)
        except Exception:
            pass
        self._losses_returned += 1
        return val

    def _pop_loss(self, block: bool) -> Optional[float]:
        eng = self.engine
        try:
            b, item = eng.losses.get(timeout=float(self.config["runtime"]["timeout_s"])) if block \
                else eng.losses.get_nowait()
        except queue.Empty:
            if block:
                eng.join(0)
                raise TimeoutError("no loss within runtime.timeout_s")
            return None
        if isinstance(item, BaseException):
            raise RuntimeError("pipeline worker failed") from item
        self._losses_returned = b
        if isinstance(item, tuple):
            host, ev = item
            ev.synchronize()
            val = float(host)
        else:
            val = float(item)
        if self._loss_publisher():
            import pickle
            self.topo.store.set(f"loss/{b}", pickle.dumps(val))
        return val

    def flush(self) -> List[float]:
        """Finish every fed batch and leave the pipeline idle but alive (the next ``feed`` refills it).
        Returns the losses not yet handed out.  Launcher mode: collective over all ranks."""
        if self.mode == "spawn":
            return self.pipeline.flush(self.last_batch_idx)
        from .runtime.engine import FlushMsg
        import threading
        done = threading.Event()
        self.engine.on_flushed = lambda b: done.set()
        self.engine.inbox.put(FlushMsg(self.last_batch_idx))
        while not done.wait(0.05):
            self._raise_if_failed()
        return self._drain_losses()

    def _drain_losses(self) -> List[float]:
        """Losses not yet handed out.  On rank 0 without the loss stage: wait until the loss stage has
        published everything up to the last fed batch."""
        rest = []
        if self._is_loss_rank():
            while True:
                l = self._pop_loss(block=False)
                if l is None:
                    break
                rest.append(l)
        elif self.rank == 0 and self.topo.replica == 0:
            while self._losses_returned < self.last_batch_idx:
                rest.append(self._remote_loss(block=True))
        return rest

    def stop(self) -> List[float]:
        """Finish every fed batch, stop the workers, and bring the final networks back.

        The reference returns only the teacher partitions to rank 0 (`tspipe/tspipe.py:466-470`); here
        the trained student comes back as well.  Returns the losses not yet handed out by ``feed``."""
        if self._stopped:
            return []
        self._stopped = True
        self.batch_q.stop()
        if self.mode == "spawn":
            return self.pipeline.stop(self.last_batch_idx)
        from .runtime.engine import StopMsg
        self._raise_if_failed()
        self.engine.inbox.put(StopMsg(self.last_batch_idx))
        while self.engine.thread.is_alive():
            self.engine.thread.join(0.1)
            self._raise_if_failed()
        self.engine.join()
        rest = self._drain_losses()
        self._collect_final()
        return rest

    def _collect_final(self) -> None:
        """Gather every stage's final state dicts on rank 0 (replica 0 only)."""
        topo = self.topo
        j = topo.stage
        mine = None
        if topo.replica == 0:
            mine = (j, _cpu_state(self.engine.online), _cpu_state(self.engine.target))
        gathered: List[Any] = [None] * topo.world
        dist.all_gather_object(gathered, mine)
        self.final_online_state: Dict[int, Dict[str, torch.Tensor]] = {}
        self.final_target_state: Dict[int, Dict[str, torch.Tensor]] = {}
        for item in gathered:
            if item is not None:
                if item[1]:
                    self.final_online_state[item[0]] = item[1]
                if item[2]:
                    self.final_target_state[item[0]] = item[2]

    def state_dicts(self) -> Tuple[Dict[int, Dict[str, torch.Tensor]], Dict[int, Dict[str, torch.Tensor]]]:
        """``(online, target)``: per-partition state dicts after :meth:`stop`."""
        if self.mode == "spawn":
            return self.pipeline.final_online_state, self.pipeline.final_target_state
        return self.final_online_state, self.final_target_state


def _cpu_state(module: nn.Module) -> Dict[str, torch.Tensor]:
    return {k: v.detach().cpu().clone() for k, v in module.state_dict().items()}


