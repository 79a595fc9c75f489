"""Configuration: the reference's YAML keys and four CLI flags, plus optional new keys.

Reference surface kept as is (`tspipe/sample_config.yaml:1-21`, `tspipe/tspipe.py:65-71,87-89`):
top-level ``tspipe`` mapping with ``train.{deferred_batch_norm,save_model_every_iter}``,
``model_split.{online,target}``, ``optimizer.{skip_optimizer,num_skip_initial_staleness,
gradient_accumulation,reduce_verbose}``, ``gpipe_emulation.{enabled,num_ubatch}``,
``async_param_update_emulation.enabled``; flags ``--tspipe-config --ip --rank --num-nodes``.

New optional keys (all defaulted so reference YAML files load unchanged):

``runtime.num_ubatch``       forward microbatches (default: stages-1, min 1, as the reference)
``runtime.bwd_split``        backward nano-batches per forward microbatch (default 2)
``runtime.dp_replicas``      data-parallel pipeline replicas (default: world / stages)
``runtime.dtype``            ``fp32`` | ``bf16`` (autocast compute, fp32 master parameters)
``runtime.backend``          ``auto`` | ``nccl`` | ``gloo``
``runtime.fused``            use the sm_100a fused kernels when on CUDA (default True)
``runtime.channels_last``    convert 4-D activations/weights to NHWC (default False)
``runtime.max_inflight``     batches the feeder may run ahead (default 3)
``runtime.prefetch``         stage-link receives posted ahead of need (default 2)
``runtime.peer_memory``      map peer GPUs' buffers for in-kernel NVLink reads (default True on CUDA)
``runtime.peer_links``       stage-boundary tensors cross through peer-mapped ring buffers with copy engines instead of
                            library send / receive kernels (default True; needs ``peer_memory``); ``runtime.link_slots``
                            = messages in flight per link (default 4)
``runtime.placement``        ``colocated`` (teacher and student stage j share rank j) | ``split`` (teacher stages
                             on the first ranks of a replica, student stages on the rest; supervised mode)
``runtime.teacher_slots``    batches the split-placement teacher may run ahead (default 2)
``runtime.resume``           checkpoint directory (or ``""``) to resume from
``runtime.fuse_ema``         fold the momentum-teacher update into the optimizer kernel when both are cut alike
``runtime.merge_views``      single stage, one microbatch: run both views of a network as one stacked forward /
                             backward with per-view BatchNorm statistics (default True)
``runtime.cuda_graphs``      replay stage forwards (teacher and student) and the student's stage backward from CUDA
                             graphs, one pair per microbatch slot, after two eager calls (default True; stages with
                             dropout, skip connections or host-side state run eagerly)
``runtime.dp_signals``       order the fused data-parallel kernels with device-side signal words in peer memory
                             (bounded waits) instead of tiny NCCL collectives (default True)
``runtime.dp_early_reduce``  start the data-parallel gradient reduction on a side stream right after the backward
                             wave, behind the look-ahead teacher forward (default True)
``runtime.sm_reserve``       SMs the persistent tensor-core kernels leave free for communication kernels
                             (default: 8 with stage links, 0 for single-stage jobs)
``runtime.heartbeat_s`` / ``runtime.timeout_s``  failure-detection heartbeat period / deadline
"""
from __future__ import annotations

import copy
from argparse import ArgumentParser, Namespace
from typing import Any, Dict, Optional, Sequence

DEFAULTS: Dict[str, Any] = {
    "train": {"deferred_batch_norm": True, "save_model_every_iter": 0},
    "model_split": {"online": None, "target": None},
    "optimizer": {"skip_optimizer": False, "num_skip_initial_staleness": 0, "gradient_accumulation": 1,
                  "reduce_verbose": False},
    "gpipe_emulation": {"enabled": False, "num_ubatch": 1},
    "async_param_update_emulation": {"enabled": False},
    "runtime": {"num_ubatch": None, "bwd_split": 2, "dp_replicas": None, "dtype": "fp32", "backend": "auto",
                "fused": True, "channels_last": False, "max_inflight": 3, "resume": "",
                "prefetch": 2, "peer_memory": True, "fuse_ema": True, "placement": "colocated", "teacher_slots": 2, "heartbeat_s": 2.0, "timeout_s": 600.0, "cuda_graphs": True, "merge_views": True, "dp_signals": True, "dp_early_reduce": True, "sm_reserve": None, "peer_links": True, "link_slots": 4},
}


def merge_config(user: Optional[Dict[str, Any]]) -> Dict[str, Any]:
    cfg = copy.deepcopy(DEFAULTS)
    for section, body in (user or {}).items():
        if section.startswith("__"):
            cfg[section] = body
            continue
        if section not in cfg:
            raise KeyError(f"unknown tspipe config section '{section}'")
        if not isinstance(body, dict):
            raise TypeError(f"tspipe config section '{section}' must be a mapping")
        for k, v in body.items():
            if k not in cfg[section]:
                raise KeyError(f"unknown tspipe config key '{section}.{k}'")
            cfg[section][k] = v
    return cfg


def load_yaml(path: str) -> Dict[str, Any]:
    import yaml
    with open(path, "r") as f:
        doc = yaml.safe_load(f)
    if not isinstance(doc, dict) or "tspipe" not in doc:
        raise KeyError(f"{path}: top-level key 'tspipe' missing")
    return merge_config(doc["tspipe"])


def parse_cli(argv: Optional[Sequence[str]] = None, required: bool = True) -> Namespace:
    """The reference's flags, read with ``parse_known_args`` so they coexist with the
    application's own parser.  Under a ``torchrun``-style launch (``RANK`` in the
    environment) ``--ip/--rank/--num-nodes`` are optional."""
    p = ArgumentParser(add_help=False)
    p.add_argument("--tspipe-config", type=str, required=required)
    p.add_argument("--ip", type=str, required=required, default="127.0.0.1")
    p.add_argument("--rank", type=int, required=required, default=0)
    p.add_argument("--num-nodes", type=int, required=required, default=1)
    args, _ = p.parse_known_args(argv)
    return args
