"""Spawn-mode workers: one process per local device, fed by the user's process.

The reference's equivalent is `tspipe/gpu_worker.py:316-355,449-466,596-600` (process per
partition, spawn context, model/optimizer/callbacks pickled to the child) plus the
scheduler-side `LocalWorker` that ships input microbatches and labels by RPC
(`:606-634`, `gpu_task.py:548-575`).  Here the parent only ships one message per batch to
each worker through a ``torch.multiprocessing`` queue (tensors travel as shared-memory
handles): the input views to stage 0, the labels to the last stage, and a bare "batch fed"
notice to the rest.
"""
from __future__ import annotations

import copy
import os
import queue
import socket
import threading
import time
import traceback
from collections import defaultdict
from typing import Any, Dict, List, Optional

import torch
import torch.multiprocessing as mp

from ..logger import Log


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_main(global_rank: int, world: int, pp: int, dp: int, cfg: Dict[str, Any], device_str: str,
                 backend: str, addr: str, port: int, payload: Dict[str, Any], inbox, outbox) -> None:
    try:
        from ..comm.topology import build_topology, init_distributed
        from ..affinity import AffinityManager
        from .engine import StageEngine
        Log.set_tag(f"w{global_rank}")
        if os.environ.get("TSPIPE_DEBUG_HANG"):
            import faulthandler
            faulthandler.dump_traceback_later(float(os.environ["TSPIPE_DEBUG_HANG"]), exit=False)
        device = torch.device(device_str)
        if device.type == "cuda":
            torch.cuda.set_device(device)
        AffinityManager.apply_for_worker(global_rank % max(world // max(cfg.get('__num_nodes', 1), 1), 1),
                                         world // max(cfg.get('__num_nodes', 1), 1))
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = addr, str(port)
        init_distributed(global_rank, world, backend, addr, port, device, cfg["runtime"]["timeout_s"])
        topo = build_topology(pp, dp, device, timeout_s=cfg["runtime"]["timeout_s"])
        engine = StageEngine(topo, cfg, payload["online"], payload["target"], payload["optimizer"],
                             payload["loss_fn"], payload["target_update_fn"], payload["momentum"],
                             kd_mode=payload["kd"], target_train_mode=payload["target_train_mode"],
                             scatter_gather_fn=payload["sg"], args=payload["args"],
                             extra_args=payload["extra_args"], inbox=inbox, ema_plan=payload["ema_plan"])
        if cfg["runtime"]["resume"]:
            from ..ckpt import load_partition
            load_partition(cfg["runtime"]["resume"], topo.stage, engine)
        every = int(cfg["train"]["save_model_every_iter"] or 0)
        art = cfg.get("__artifact_dir", "")

        def on_done(b: int) -> None:
            outbox.put(("done", global_rank, b))
            if every > 0 and b % every == 0 and art:
                from ..ckpt import save_partition
                save_partition(art, b, topo.stage, engine, replica=topo.replica)
        engine.on_batch_done = on_done
        engine.on_flushed = lambda b: outbox.put(("flushed", global_rank, b))

        stop_fwd = threading.Event()

        def forward_losses() -> None:
            while not (stop_fwd.is_set() and engine.losses.empty()):
                try:
                    b, item = engine.losses.get(timeout=0.05)
                except queue.Empty:
                    continue
                if isinstance(item, tuple):
                    host, ev = item
                    ev.synchronize()
                    item = float(host)
                outbox.put(("loss", b, item))
        fwd = threading.Thread(target=forward_losses, daemon=True)
        if topo.is_last and topo.replica == 0:
            fwd.start()
        outbox.put(("ready", global_rank, None))
        engine.run()
        stop_fwd.set()
        if fwd.is_alive():
            fwd.join()
        state = None
        if topo.replica == 0:
            state = ({k: v.detach().cpu() for k, v in engine.online.state_dict().items()},
                     {k: v.detach().cpu() for k, v in engine.target.state_dict().items()})
        if state is not None:       # as bytes: shared-memory handles would die with this process
            import io
            buf = io.BytesIO()
            torch.save(state, buf)
            state = buf.getvalue()
        outbox.put(("final", topo.stage, state))
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    except BaseException as e:  # noqa: BLE001 - surfaced in the parent
        outbox.put(("error", global_rank, f"{e!r}\n{traceback.format_exc()}"))
        raise


class SpawnedPipeline:
    def __init__(self, tsp, device, pp_total: Optional[int]):
        from ..tspipe import TSPipeMode
        cfg = tsp.config
        args = tsp.args
        use_cuda = torch.cuda.is_available() and cfg["runtime"]["backend"] != "gloo" and \
            (device is None or torch.device(device).type == "cuda")
        n_nodes = int(args.num_nodes)
        if use_cuda:
            local = torch.cuda.device_count()
        else:
            if pp_total is None:
                raise ValueError("model_split is required to size a CPU pipeline")
            dp_cfg = cfg["runtime"]["dp_replicas"] or 1
            local = pp_total * dp_cfg // n_nodes
        world = local * n_nodes
        pp = pp_total or world // (cfg["runtime"]["dp_replicas"] or 1)
        dp = cfg["runtime"]["dp_replicas"] or world // pp
        if pp * dp != world:
            raise ValueError("The number of GPUs and the number of partitions must match "
                             f"(world {world}, partitions {pp}, dp_replicas {dp}).")
        self.pp, self.dp, self.world, self.local = pp, dp, world, local
        backend = cfg["runtime"]["backend"]
        if backend == "auto":
            backend = "nccl" if use_cuda else "gloo"
        tsp._build_partitions(pp)
        gp, rt = cfg["gpipe_emulation"], cfg["runtime"]
        self.n_ubatch = gp["num_ubatch"] if gp["enabled"] else (rt["num_ubatch"] or max(pp - 1, 1))
        self.bwd_split = 1 if gp["enabled"] else rt["bwd_split"]
        cfg["__num_nodes"] = n_nodes
        port = int(os.environ.get("TSPIPE_PORT", 0)) or (31101 if n_nodes > 1 else _free_port())
        ctx = mp.get_context("spawn")
        self.outbox = ctx.Queue()
        self.inboxes: Dict[int, Any] = {}
        self.procs: List[Any] = []
        self.first_rank_local: List[int] = []
        self.last_rank_local: List[int] = []
        kd = tsp.tspipe_mode == TSPipeMode.SUPERVISED_MOMENTUM
        for w in range(local):
            g = args.rank * local + w
            stage, replica = g % pp, g // pp
            part_on, part_tg = tsp.partitions_online[stage], tsp.partitions_target[stage]
            if replica > 0:
                part_on, part_tg = copy.deepcopy(part_on), copy.deepcopy(part_tg)
            opt = _optimizer_shell(tsp.optimizer, tsp.partitions_online[stage], part_on)
            payload = dict(online=part_on, target=part_tg, optimizer=opt, loss_fn=tsp.loss_fn,
                           target_update_fn=tsp.target_update_fn, momentum=tsp.momentum, kd=kd,
                           target_train_mode=tsp.target_train_mode, sg=tsp.scatter_gather_fn,
                           args=tsp.args, extra_args=tsp.extra_args,
                           ema_plan=tsp.ema_plans[stage] if tsp.ema_plans else None)
            inbox = ctx.Queue()
            dev = f"cuda:{w}" if use_cuda else "cpu"
            p = ctx.Process(target=_worker_main, daemon=True,
                            args=(g, world, pp, dp, cfg, dev, backend, args.ip, port, payload, inbox, self.outbox))
            p.start()
            self.inboxes[g] = inbox
            self.procs.append(p)
        self.losses: "queue.Queue" = queue.Queue()
        self.done: Dict[int, int] = defaultdict(int)
        self.finals: Dict[int, Any] = {}
        self.flushed: Dict[int, int] = {}
        self.final_online_state: Dict[int, Any] = {}
        self.final_target_state: Dict[int, Any] = {}
        self._losses_returned = 0
        ready = 0
        while ready < local:
            kind, a, b = self._next_event(timeout=cfg["runtime"]["timeout_s"])
            if kind == "ready":
                ready += 1

    # -- events from the workers --------------------------------------------------------------------
    def _next_event(self, timeout: float):
        deadline = time.monotonic() + timeout
        while True:
            try:
                ev = self.outbox.get(timeout=0.2)
            except queue.Empty:
                for p in self.procs:
                    if not p.is_alive() and p.exitcode not in (0, None):
                        raise RuntimeError(f"pipeline worker pid {p.pid} exited with code {p.exitcode}")
                if time.monotonic() > deadline:
                    raise TimeoutError("no event from the pipeline workers within runtime.timeout_s")
                continue
            kind = ev[0]
            if kind == "error":
                raise RuntimeError(f"pipeline worker {ev[1]} failed: {ev[2]}")
            if kind == "loss":
                self.losses.put((ev[1], ev[2]))
            elif kind == "done":
                self.done[ev[1]] = ev[2]
            elif kind == "final":
                self.finals[ev[1]] = ev[2]
            elif kind == "flushed":
                self.flushed[ev[1]] = ev[2]
            return ev

    def _drain_events(self) -> None:
        while True:
            try:
                ev = self.outbox.get_nowait()
            except queue.Empty:
                return
            if ev[0] == "error":
                raise RuntimeError(f"pipeline worker {ev[1]} failed: {ev[2]}")
            if ev[0] == "loss":
                self.losses.put((ev[1], ev[2]))
            elif ev[0] == "done":
                self.done[ev[1]] = ev[2]
            elif ev[0] == "final":
                self.finals[ev[1]] = ev[2]
            elif ev[0] == "flushed":
                self.flushed[ev[1]] = ev[2]

    # -- feeding --------------------------------------------------------------------------------------
    def submit(self, msg, views: List[Any], labels: Any) -> None:
        from ..utils import pytree as pt
        max_inflight = int(self.cfg_max_inflight(msg))
        while self.inboxes and msg.batch_id - min(self.done[g] for g in self.inboxes) > max_inflight:
            self._next_event(timeout=self._timeout)
        for g, inbox in self.inboxes.items():
            stage, replica = g % self.pp, g // self.pp
            m = copy.copy(msg)
            if stage == 0:
                m.views = [_replica_slice(v, replica, self.dp) for v in views]
            if stage == self.pp - 1:
                m.labels = _replica_slice(labels, replica, self.dp) if labels is not None else None
            inbox.put(m)

    def broadcast(self, msg) -> None:
        for inbox in self.inboxes.values():
            inbox.put(msg)

    _timeout = 600.0

    def cfg_max_inflight(self, msg) -> int:
        return getattr(self, "max_inflight", 3)

    def poll_loss(self, last_fed: int, max_inflight: int) -> Optional[float]:
        self.max_inflight = max_inflight
        self._drain_events()
        block = last_fed - self._losses_returned >= max_inflight
        while True:
            try:
                b, l = self.losses.get_nowait()
                self._losses_returned = b
                return l
            except queue.Empty:
                if not block:
                    return None
                self._next_event(timeout=self._timeout)

    def flush(self, last_batch: int) -> List[float]:
        from .engine import FlushMsg
        self.broadcast(FlushMsg(last_batch))
        while any(self.flushed.get(g, -1) < last_batch for g in self.inboxes):
            self._next_event(timeout=self._timeout)
        self._drain_events()
        rest = []
        while not self.losses.empty():
            b, l = self.losses.get()
            self._losses_returned = b
            rest.append(l)
        return rest

    def stop(self, last_batch: int) -> List[float]:
        from .engine import StopMsg
        for inbox in self.inboxes.values():
            inbox.put(StopMsg(last_batch))
        while len(self.finals) < len({g % self.pp for g in self.inboxes}) or \
                any(self.done[g] < last_batch for g in self.inboxes):
            self._next_event(timeout=self._timeout)
        for p in self.procs:
            p.join(timeout=60)
        self._drain_events()
        rest = []
        while not self.losses.empty():
            rest.append(self.losses.get()[1])
        for stage, st in self.finals.items():
            if st is not None:
                import io
                self.final_online_state[stage], self.final_target_state[stage] = torch.load(io.BytesIO(st))
        return rest

    def join(self) -> None:
        for p in self.procs:
            p.join()


def _replica_slice(obj: Any, replica: int, dp: int) -> Any:
    if dp == 1 or obj is None:
        return obj
    from ..utils import pytree as pt
    return pt.generic_scatter(obj, dp)[replica]


def _optimizer_shell(optimizer, src_partition, dst_partition):
    """A copy of the user's optimizer that owns only ``dst_partition``'s parameters, with every
    param group's hyper-parameters kept (`tspipe/tspipe.py:169-180`)."""
    if optimizer is None:
        return None
    src = list(src_partition.parameters())
    dst = list(dst_partition.parameters())
    mapping = {id(s): d for s, d in zip(src, dst)}
    shell = copy.copy(optimizer)
    shell.state = defaultdict(dict)
    shell.param_groups = []
    for g in optimizer.param_groups:
        ng = {k: v for k, v in g.items() if k != "params"}
        ng["params"] = [mapping[id(p)] for p in g["params"] if id(p) in mapping]
        shell.param_groups.append(ng)
    return shell
