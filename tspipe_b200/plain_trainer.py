"""The non-pipelined trainer of the reference applications, behind the :class:`~tspipe_b200.TSPipe` interface.

The reference scripts carry a plain single-device training loop next to the pipelined one
(`benchmarks/byol/trainer.py:21-157` ``BYOLTrainer``, the non-``--tspipe`` branches of
`benchmarks/moco-v3/main.py:396-446` and `benchmarks/soft_target/train_kd.py:366-420`): teacher forward without
gradient, student forward, loss, backward, optimizer step, momentum update of the teacher - no delay, no microbatches.
It is what a loss curve of the pipelined run is compared against.  :class:`PlainTrainer` has the methods the
applications use on ``TSPipe`` (``feed``, ``feed_epoch``, ``update_lr``, ``update_momentum``, ``stop``,
``state_dicts``, ``is_primary``, ``meter``), so every application runs either way (``--plain``).

``feed`` returns the loss of the batch it was given (the pipelined ``feed`` returns the loss of an earlier batch).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
from torch import nn

from .batch_ops import ScatterGatherFn, defaultScatterGatherFn
from .run_log import ThroughputMeter
from .utils import pytree as pt


class PlainTrainer:
    def __init__(self, module_online: nn.Sequential, module_target: nn.Sequential,
                 module_predictor: Optional[nn.Sequential], optimizer: torch.optim.Optimizer, loss_fn: Callable,
                 target_update_fn: Optional[Callable], momentum: float, artifact_dir: str = "", *,
                 supervised: bool = False, target_train_mode: bool = True,
                 scatter_gather_fn: ScatterGatherFn = defaultScatterGatherFn, args: Any = None, extra_args: Any = None,
                 device: Optional[torch.device] = None, dtype: str = "fp32"):
        self.device = torch.device(device) if device is not None else \
            torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
        children = list(module_online.children()) + (list(module_predictor.children()) if module_predictor is not None
                                                     else [])
        self.online = nn.Sequential(*children).to(self.device).train()
        self.target = module_target.to(self.device).train(target_train_mode)
        for p in self.target.parameters():
            p.requires_grad_(False)
        self.n_shared = len(list(module_online.parameters()))      # the predictor has no teacher counterpart
        self.optimizer, self.loss_fn, self.update_fn = optimizer, loss_fn, target_update_fn
        self.momentum, self.supervised = float(momentum), bool(supervised)
        self.args, self.extra_args, self.sg = args, extra_args, scatter_gather_fn
        self.autocast = dtype == "bf16"
        self.epoch, self.batches = 0, 0
        self.meter = ThroughputMeter()
        self._stopped = False

    # -- the TSPipe surface the applications use -------------------------------------------------------
    def is_primary(self) -> bool:
        return True

    def update_lr(self, lr) -> None:
        lrs = lr if isinstance(lr, (list, tuple)) else [lr] * len(self.optimizer.param_groups)
        for g, v in zip(self.optimizer.param_groups, lrs):
            g["lr"] = v

    def update_momentum(self, momentum: float) -> None:
        self.momentum = float(momentum)

    def feed_epoch(self) -> None:
        self.epoch += 1

    def _to_device(self, x: Any) -> Any:
        return pt.tree_map_tensors(lambda t: t.to(self.device, non_blocking=True), x)

    def _amp(self):
        return torch.autocast(device_type=self.device.type, dtype=torch.bfloat16, enabled=self.autocast)

    def feed(self, view_1: Any, view_2: Any, view_target: Any = None) -> float:
        assert not self._stopped, "trainer already stopped"
        self.meter.add(self.sg.batch_size(view_1))
        v1, v2 = self._to_device(view_1), self._to_device(view_2)
        with self._amp():
            if self.supervised:
                assert view_target is not None, "Supervised learning requires labels."
                with torch.no_grad():
                    t = pt.unwrap(self.target(v2))
                o = pt.unwrap(self.online(v1))
                loss = self.loss_fn(o, t, self._to_device(view_target), self.args, self.extra_args, self.epoch)
            else:
                assert view_target is None, "Self-supervised learning does not support labels."
                with torch.no_grad():
                    t1, t2 = pt.unwrap(self.target(v1)), pt.unwrap(self.target(v2))
                o1, o2 = pt.unwrap(self.online(v1)), pt.unwrap(self.online(v2))
                loss = self.loss_fn(o1, o2, t1, t2, self.args, self.extra_args)
        self.optimizer.zero_grad(set_to_none=True)
        loss.backward()
        self.optimizer.step()
        if self.update_fn is not None:
            with torch.no_grad():
                online = [p.detach() for p in self.online.parameters()][: self.n_shared]
                new = self.update_fn(self.momentum, online, list(self.target.parameters()))
                for p, v in zip(self.target.parameters(), new):
                    if v is not p:
                        p.copy_(v)
        self.batches += 1
        return float(loss.detach())

    def stop(self) -> List[float]:
        self._stopped = True
        return []

    def state_dicts(self) -> Tuple[Dict[int, Dict[str, torch.Tensor]], Dict[int, Dict[str, torch.Tensor]]]:
        cpu = lambda m: {k: v.detach().cpu().clone() for k, v in m.state_dict().items()}
        return {0: cpu(self.online)}, {0: cpu(self.target)}
