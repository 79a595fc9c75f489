#!/usr/bin/env python
"""Soft-target knowledge distillation with a frozen teacher (`benchmarks/soft_target/train_kd.py:215-227,
439-461` in the reference): teacher forward-only, student trained with
``CE + lambda_kd * T^2 * KL(softmax(t/T) || softmax(s/T))`` (`kd_losses/st.py:18-23`, `train_kd.py:448-453`).

    torchrun --nproc-per-node 8 benchmarks/soft_target/train_kd.py --tspipe-config benchmarks/soft_target/tspipe.yaml \
        --t-name vit_large --s-name vit_base --batch-size 2048 --dummy

Models come from :func:`create_model` (`benchmarks/soft_target/models/factory.py:20-30`): ``vit_*`` or
``resnet*`` classifiers as flat sequentials.
"""
from __future__ import annotations

import argparse
import os
import sys
from argparse import Namespace

import torch
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tspipe_b200 import TSPipe, TSPipeMode  # noqa: E402
from tspipe_b200.losses import logits_kd, soft_target_kd  # noqa: E402
from tspipe_b200.models.resnet import resnet_trunk_children, trunk_width  # noqa: E402
from tspipe_b200.models.vit import vit_classifier  # noqa: E402
from tspipe_b200.optim import SGD, AdamW  # noqa: E402
from tspipe_b200.plain_trainer import PlainTrainer  # noqa: E402
from tspipe_b200.run_log import RunLog  # noqa: E402


def create_model(name: str, num_classes: int) -> nn.Sequential:
    if name.startswith("vit"):
        return vit_classifier(name, num_classes)
    if name.startswith("efficientnet"):
        from tspipe_b200.models.efficientnet import EfficientNet
        return EfficientNet(name, num_classes).to_sequential()
    if name.startswith("resnet"):
        ch = resnet_trunk_children(name)
        ch["fc"] = nn.Linear(trunk_width(name), num_classes)
        return nn.Sequential(ch)
    raise ValueError(f"unknown model {name}")


def dummy_target_update(m, online, target):
    return target


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--t-name", default="vit_large")
    ap.add_argument("--s-name", default="vit_base")
    ap.add_argument("--num-class", type=int, default=1000)
    ap.add_argument("--batch-size", type=int, default=2048)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--iters-per-epoch", type=int, default=30)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "sgd"])
    ap.add_argument("--kd-mode", default="st", choices=["st", "logits"])
    ap.add_argument("--T", type=float, default=4.0)
    ap.add_argument("--lambda-kd", type=float, default=1.0)
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--dummy", action="store_true", default=True)
    ap.add_argument("--artifact-dir", default="runs/soft_target")
    ap.add_argument("--plain", action="store_true", help="the reference's non-pipelined trainer (one device)")
    args, _ = ap.parse_known_args()

    tnet, snet = create_model(args.t_name, args.num_class), create_model(args.s_name, args.num_class)
    opt = AdamW(snet.parameters(), lr=args.lr, weight_decay=0.05) if args.optimizer == "adamw" else \
        SGD(snet.parameters(), lr=args.lr, momentum=0.9, weight_decay=1e-4, nesterov=True)
    loss_fn = soft_target_kd if args.kd_mode == "st" else logits_kd
    if args.plain:
        tsp = PlainTrainer(snet, tnet, None, opt, loss_fn, None, 1.0, args.artifact_dir, supervised=True,
                           target_train_mode=False, extra_args=Namespace(T=args.T, lambda_kd=args.lambda_kd))
    else:
        tsp = TSPipe(snet, tnet, None, opt, loss_fn, None, 1.0, args.artifact_dir,
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False,
                     extra_args=Namespace(T=args.T, lambda_kd=args.lambda_kd))
    g = torch.Generator().manual_seed(0)
    img = torch.randn(args.batch_size, 3, args.image, args.image, generator=g)
    lab = torch.randint(0, args.num_class, (args.batch_size,), generator=g)
    if torch.cuda.is_available():
        img, lab = img.pin_memory(), lab.pin_memory()
    log = RunLog(args.artifact_dir, enabled=tsp.is_primary())      # TensorBoard scalars + scalars.csv + model.pth
    niter = 0
    for epoch in range(args.epochs):
        for _ in range(args.iters_per_epoch):
            loss = tsp.feed(img, img, lab)
            niter += 1
            if loss is not None:
                log.scalar("loss", loss, niter)
                if niter % 10 == 0 and tsp.is_primary():
                    print(f"iter {niter} loss {loss:.4f} {tsp.meter.recent():.1f} samples/s", flush=True)
        tsp.feed_epoch()
        log.scalar("samples_per_second", tsp.meter.overall(), niter)
    for k, loss in enumerate(tsp.stop()):
        log.scalar("loss", loss, niter + 1 + k)
    log.save_final(tsp, opt)
    log.close()


if __name__ == "__main__":
    main()
