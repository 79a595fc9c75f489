#!/usr/bin/env python
"""MoCo-v3 pre-training of a ViT with the pipelined runtime (`benchmarks/moco-v3/main.py:358-367,448-476`).

    torchrun --nproc-per-node 8 benchmarks/moco_v3/main.py --tspipe-config benchmarks/moco_v3/tspipe.yaml \
        --arch vit_base --batch-size 4096 --dummy

Learning rate and momentum are re-scheduled every iteration as in the reference
(`main.py:534-548`): ``lr = base * bs/256`` with linear warm-up and half-cosine decay, momentum
``m -> 1`` along a half cosine.  With data-parallel pipeline replicas (``runtime.dp_replicas``) the keys
of all replicas are gathered through peer memory before the contrastive logits
(:mod:`tspipe_b200.parallel.keys`), the path the reference disables in its pipeline mode
(`main.py:154,159`).
"""
from __future__ import annotations

import argparse
import math
import os
import sys
from argparse import Namespace

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tspipe_b200 import TSPipe  # noqa: E402
from tspipe_b200.dataloader import DummyInputGenerator, FastDataLoader  # noqa: E402
from tspipe_b200.losses import ema_update, moco_loss  # noqa: E402
from tspipe_b200.models.vit import moco_vit_networks  # noqa: E402
from tspipe_b200.optim import LARS, AdamW  # noqa: E402
from tspipe_b200.plain_trainer import PlainTrainer  # noqa: E402
from tspipe_b200.run_log import RunLog  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="vit_base")
    ap.add_argument("--batch-size", type=int, default=4096)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--warmup-epochs", type=int, default=0)
    ap.add_argument("--lr", type=float, default=1.5e-4)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "lars"])
    ap.add_argument("--moco-dim", type=int, default=256)
    ap.add_argument("--moco-mlp-dim", type=int, default=4096)
    ap.add_argument("--moco-m", type=float, default=0.99)
    ap.add_argument("--moco-m-cos", action="store_true", default=True)
    ap.add_argument("--moco-t", type=float, default=0.2)
    ap.add_argument("--stop-grad-conv1", action="store_true")
    ap.add_argument("--data", default="")
    ap.add_argument("--dummy", action="store_true")
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--max-iters", type=int, default=0)
    ap.add_argument("--artifact-dir", default="runs/moco_v3")
    ap.add_argument("--plain", action="store_true",
                    help="the reference's non-pipelined trainer (one device, immediate momentum encoder)")
    args, _ = ap.parse_known_args()

    base, momentum, predictor = moco_vit_networks(args.arch, args.moco_dim, args.moco_mlp_dim, args.stop_grad_conv1)
    params = [p for p in list(base.parameters()) + list(predictor.parameters())]
    lr = args.lr * args.batch_size / 256
    opt = AdamW(params, lr=lr, weight_decay=args.weight_decay) if args.optimizer == "adamw" else \
        LARS(params, lr=lr, weight_decay=args.weight_decay, momentum=0.9)
    if args.plain:
        tsp = PlainTrainer(base, momentum, predictor, opt, moco_loss, ema_update, args.moco_m, args.artifact_dir,
                           extra_args=Namespace(moco_t=args.moco_t))
    else:
        tsp = TSPipe(base, momentum, predictor, opt, moco_loss, ema_update, args.moco_m, args.artifact_dir,
                     extra_args=Namespace(moco_t=args.moco_t))
    if args.dummy or not args.data:
        loader = DummyInputGenerator(args.batch_size, input_shape=args.image, pin=torch.cuda.is_available())
    else:
        from tspipe_b200.datasets import two_crop_imagefolder
        loader = FastDataLoader(two_crop_imagefolder(args.data), batch_size=args.batch_size, shuffle=True,
                                num_workers=16, drop_last=True)
    iters_per_epoch = len(loader)
    log = RunLog(args.artifact_dir, enabled=tsp.is_primary())      # TensorBoard scalars + scalars.csv + model.pth
    niter = 0
    for epoch in range(args.epochs):
        for i, ((v1, v2), _) in enumerate(loader):
            e = epoch + i / iters_per_epoch
            if e < args.warmup_epochs:
                cur_lr = lr * e / max(args.warmup_epochs, 1)
            else:
                cur_lr = lr * 0.5 * (1 + math.cos(math.pi * (e - args.warmup_epochs) /
                                                  max(args.epochs - args.warmup_epochs, 1)))
            tsp.update_lr(cur_lr)
            if args.moco_m_cos:
                tsp.update_momentum(1 - 0.5 * (1 + math.cos(math.pi * e / args.epochs)) * (1 - args.moco_m))
            loss = tsp.feed(v1, v2)
            niter += 1
            if loss is not None:
                log.scalar("loss", loss, niter)
                if niter % 10 == 0 and tsp.is_primary():
                    print(f"iter {niter} loss {loss:.4f} {tsp.meter.recent():.1f} img/s", flush=True)
            if args.max_iters and niter >= args.max_iters:
                break
        tsp.feed_epoch()
        log.scalar("learning_rate", cur_lr, niter)
        log.scalar("images_per_second", tsp.meter.overall(), niter)
        if args.max_iters and niter >= args.max_iters:
            break
    for k, loss in enumerate(tsp.stop()):
        log.scalar("loss", loss, niter + 1 + k)
    log.save_final(tsp, opt)
    log.close()


if __name__ == "__main__":
    main()
