#!/usr/bin/env python
"""BYOL pre-training with the pipelined runtime (`benchmarks/byol/main.py`, `trainer.py:214-280` in the
reference).

    torchrun --nproc-per-node 2 benchmarks/byol/main.py --tspipe-config benchmarks/byol/tspipe.yaml
    python benchmarks/byol/main.py --tspipe-config=benchmarks/byol/tspipe.yaml --ip=localhost --rank=0 --num-nodes=1

``trainer.dummy_input: True`` feeds synthetic views (throughput runs); otherwise ``dataset.path`` must hold
an ImageFolder tree.
"""
from __future__ import annotations

import argparse
import ast
import os
import sys

import torch
import yaml

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tspipe_b200 import TSPipe  # noqa: E402
from tspipe_b200.dataloader import DummyInputGenerator, FastDataLoader  # noqa: E402
from tspipe_b200.losses import byol_loss, ema_update  # noqa: E402
from tspipe_b200.models.resnet import byol_networks  # noqa: E402
from tspipe_b200.optim import LARS, SGD, AdamW  # noqa: E402
from tspipe_b200.plain_trainer import PlainTrainer  # noqa: E402
from tspipe_b200.profiler import TSPipeProfiler  # noqa: E402
from tspipe_b200.run_log import RunLog  # noqa: E402
from tspipe_b200.schedules import cosine_lr, cosine_momentum  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=os.path.join(os.path.dirname(__file__), "config.yaml"))
    ap.add_argument("--artifact-dir", default="runs/byol")
    ap.add_argument("--max-iters", type=int, default=0)
    ap.add_argument("--plain", action="store_true",
                    help="the reference's non-pipelined trainer (one device, immediate teacher) for loss-curve comparison")
    args, _ = ap.parse_known_args()
    cfg = yaml.safe_load(open(args.config))
    head = cfg["network"]["projection_head"]
    online, target, predictor = byol_networks(cfg["network"]["name"], head["mlp_hidden_size"], head["projection_size"])
    params = list(online.parameters()) + list(predictor.parameters())
    opt_cls = {"lars": LARS, "sgd": SGD, "adamw": AdamW}[cfg["trainer"]["optimizer_type"]]
    opt_args = dict(cfg["optimizer"]["params"])
    bs = cfg["trainer"]["batch_size"]
    if opt_cls is LARS:
        opt_args["lr"] = opt_args["lr"] * bs / 256
    elif opt_cls is AdamW:
        opt_args.pop("momentum", None)
    optimizer = opt_cls(params, **opt_args)
    m0, epochs = cfg["trainer"]["m"], cfg["trainer"]["max_epochs"]
    with TSPipeProfiler(filename=os.path.join(args.artifact_dir, "profile_out.csv")) as prof:
        if args.plain:
            tsp = PlainTrainer(online, target, predictor, optimizer, byol_loss, ema_update, m0, args.artifact_dir)
        else:
            tsp = TSPipe(online, target, predictor, optimizer, byol_loss, ema_update, m0, args.artifact_dir,
                         profiler=prof)
        if cfg["trainer"]["dummy_input"]:
            image = ast.literal_eval(cfg["data_transforms"]["input_shape"])[0]
            loader = DummyInputGenerator(bs, input_shape=image, pin=torch.cuda.is_available())
        else:
            from tspipe_b200.datasets import two_crop_imagefolder
            loader = FastDataLoader(two_crop_imagefolder(cfg["dataset"]["path"], cfg["dataset"]["name"]), batch_size=bs,
                                    num_workers=cfg["trainer"]["num_workers"], shuffle=True, drop_last=True)
        base_lr = optimizer.param_groups[0]["lr"]
        log = RunLog(args.artifact_dir, enabled=tsp.is_primary())      # TensorBoard scalars + scalars.csv + model.pth
        niter = 0
        for epoch in range(epochs):
            for (v1, v2), _ in loader:
                loss = tsp.feed(v1, v2)
                niter += 1
                if loss is not None:
                    log.scalar("loss", loss, niter)
                    if niter % 10 == 0 and tsp.is_primary():
                        print(f"iter {niter} loss {loss:.4f} {tsp.meter.recent():.1f} img/s", flush=True)
                if args.max_iters and niter >= args.max_iters:
                    break
            tsp.feed_epoch()
            lr, m = cosine_lr(epoch + 1, epochs, base_lr), cosine_momentum(epoch, epochs, m0)
            tsp.update_lr(lr)
            tsp.update_momentum(m)
            log.scalar("learning_rate", lr, niter)
            log.scalar("momentum", m, niter)
            log.scalar("images_per_second", tsp.meter.overall(), niter)
            if args.max_iters and niter >= args.max_iters:
                break
        for k, loss in enumerate(tsp.stop()):        # losses of the batches still in flight
            log.scalar("loss", loss, niter + 1 + k)
        log.save_final(tsp, optimizer)           # model.pth: online / target / optimizer state dicts
        log.close()


if __name__ == "__main__":
    main()
