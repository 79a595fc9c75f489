"""Checkpoint files in the reference's per-partition format, plus resume.

Format (`tspipe/gpu_task.py:726-734`): ``{artifact_dir}/model_batch{B}_part{P}.pt`` holding
``online_network_state_dict``, ``target_network_state_dict`` and ``optimizer_state_dict``, the
state-dict keys being the child names of the user's ``nn.Sequential`` that fell into partition
``P``.  Extra keys written here (ignored by the reference's readers): ``tspipe_b200`` with the
batch id, the momentum, the gradient-accumulation counter and the deferred-BatchNorm counters
(per layer, and the flat accumulators of a partition's :class:`~tspipe_b200.batchnorm.BatchNormGroup`),
which is what resuming needs (the reference cannot resume a pipeline run,
`benchmarks/moco-v3/main.py:284-286`).

Data-parallel replicas: with the fused reduce-scatter + step kernels every replica updates, and therefore
holds, only its ``1/R`` range of the flat optimizer state.  Replica 0 writes the partition file as above;
every replica (0 included) also writes ``model_batch{B}_part{P}_dp{r}.pt`` with its own range
``[lo, hi)`` of every state buffer.  On load each replica reads all ``_dp*.pt`` files of the batch and
reassembles the complete state, so a run may resume with a different replica count.
"""
from __future__ import annotations

import glob
import os
import re
from typing import Any, Dict, Optional

import torch

from .batchnorm import DeferredBatchNorm


def partition_path(artifact_dir: str, batch_id: int, partition_id: int) -> str:
    return os.path.join(artifact_dir, f"model_batch{batch_id}_part{partition_id}.pt")


def _bn_counters(module: torch.nn.Module) -> Dict[str, Any]:
    return {name: (m.counter, m.tracked) for name, m in module.named_modules() if isinstance(m, DeferredBatchNorm)}


def _set_bn_counters(module: torch.nn.Module, counters: Dict[str, Any]) -> None:
    for name, m in module.named_modules():
        if isinstance(m, DeferredBatchNorm) and name in counters:
            m.counter, m.tracked = counters[name]


def shard_path(artifact_dir: str, batch_id: int, partition_id: int, replica: int) -> str:
    return os.path.join(artifact_dir, f"model_batch{batch_id}_part{partition_id}_dp{replica}.pt")


def _atomic_save(blob: Any, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(blob, tmp)
    os.replace(tmp, path)


def _group_state(engine) -> Dict[str, Any]:
    out = {}
    for name in ("bn_group_online", "bn_group_target"):
        g = getattr(engine, name, None)
        if g is not None and getattr(g, "layers", None):
            out[name] = {"acc": g._acc.detach().cpu().clone(), "tracked": int(g.tracked)}
    return out


def _set_group_state(engine, state: Dict[str, Any]) -> None:
    for name, st in state.items():
        g = getattr(engine, name, None)
        if g is not None and getattr(g, "layers", None) and tuple(st["acc"].shape) == tuple(g._acc.shape):
            with torch.no_grad():
                g._acc.copy_(st["acc"])
            g.tracked = int(st["tracked"])


def save_partition(artifact_dir: str, batch_id: int, partition_id: int, engine, replica: int = 0) -> Optional[str]:
    """Write this stage's shard.  Replica 0 writes the partition file (replicas hold identical model states);
    when the optimizer state is sharded over the replicas, every replica writes its own range next to it."""
    os.makedirs(artifact_dir, exist_ok=True)
    if engine.cuda:
        engine.compute.synchronize()
    opt = engine.optimizer
    shard = getattr(opt, "flat_shard_state", None)
    if shard is not None:
        piece = shard()
        if piece is not None:
            _atomic_save(piece, shard_path(artifact_dir, batch_id, partition_id, replica))
    if replica != 0:
        return None
    blob = {
        "online_network_state_dict": engine.online.state_dict(),
        "target_network_state_dict": engine.target.state_dict(),
        "optimizer_state_dict": opt.state_dict() if opt is not None else None,
        "tspipe_b200": {"batch_id": batch_id, "momentum": engine.momentum, "ga_count": engine.ga_count,
                        "bn_online": _bn_counters(engine.online), "bn_target": _bn_counters(engine.target),
                        "bn_groups": _group_state(engine)},
    }
    path = partition_path(artifact_dir, batch_id, partition_id)
    _atomic_save(blob, path)
    return path


def latest_batch(artifact_dir: str, partition_id: int) -> Optional[int]:
    best = None
    for f in glob.glob(os.path.join(artifact_dir, f"model_batch*_part{partition_id}.pt")):
        m = re.search(r"model_batch(\d+)_part\d+\.pt$", f)
        if m:
            best = max(best or 0, int(m.group(1)))
    return best


def load_partition(path_or_dir: str, partition_id: int, engine, batch_id: Optional[int] = None) -> int:
    """Restore a stage from its shard (the latest one in a directory unless ``batch_id`` is given).
    Returns the batch id the shard was written at."""
    if os.path.isdir(path_or_dir):
        b = batch_id if batch_id is not None else latest_batch(path_or_dir, partition_id)
        if b is None:
            raise FileNotFoundError(f"no checkpoint for partition {partition_id} in {path_or_dir}")
        path = partition_path(path_or_dir, b, partition_id)
    else:
        path = path_or_dir
    blob = torch.load(path, map_location=engine.device, weights_only=False)
    with torch.no_grad():
        engine.online.load_state_dict(blob["online_network_state_dict"])
        engine.target.load_state_dict(blob["target_network_state_dict"])
    extra = blob.get("tspipe_b200", {})
    if engine.optimizer is not None and blob.get("optimizer_state_dict") is not None:
        engine.optimizer.load_state_dict(blob["optimizer_state_dict"])
        merge = getattr(engine.optimizer, "load_flat_shards", None)
        if merge is not None:
            b = int(extra.get("batch_id", 0))
            pieces = sorted(glob.glob(os.path.join(os.path.dirname(path),
                                                   f"model_batch{b}_part{partition_id}_dp*.pt")))
            if pieces:
                merge([torch.load(f, map_location="cpu", weights_only=False) for f in pieces])
    engine.momentum = extra.get("momentum", engine.momentum)
    engine.ga_count = extra.get("ga_count", 0)
    _set_bn_counters(engine.online, extra.get("bn_online", {}))
    _set_bn_counters(engine.target, extra.get("bn_target", {}))
    _set_group_state(engine, extra.get("bn_groups", {}))
    return int(extra.get("batch_id", 0))
