#!/usr/bin/env python
"""DistilBERT-style masked-LM distillation (`benchmarks/distilbert/train.py`, `distiller.py:622-772` in the
reference): BERT teacher forward-only, student with half the layers, loss
``5.0 * KL(T=2) + 2.0 * MLM-CE + 1.0 * cosine(hidden)``, AdamW(betas 0.9/0.98, eps 1e-6), linear warm-up /
decay, 15 % MLM masking with the 80/10/10 rule (`distiller.py:194-257`).

    torchrun --nproc-per-node 4 benchmarks/distilbert/train.py --tspipe-config benchmarks/distilbert/tspipe.yaml

Batches are dicts ``{"input_ids", "attention_mask"}``; a custom :class:`ScatterGatherFn` splits them into
microbatches (`distiller.py:648-652,774-836`).  Token ids are synthetic (uniform in ``[1000, vocab)``).
"""
from __future__ import annotations

import argparse
import os
import sys
from argparse import Namespace

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tspipe_b200 import ScatterGatherFn, TSPipe, TSPipeMode  # noqa: E402
from tspipe_b200.batch_ops import Batch  # noqa: E402
from tspipe_b200.losses import distil_loss  # noqa: E402
from tspipe_b200.models import bert as B  # noqa: E402
from tspipe_b200.optim import AdamW  # noqa: E402
from tspipe_b200.plain_trainer import PlainTrainer  # noqa: E402
from tspipe_b200.run_log import RunLog  # noqa: E402
from tspipe_b200.schedules import linear_warmup_decay  # noqa: E402
from tspipe_b200.utils import pytree as pt  # noqa: E402


def dict_scatter(obj, chunks):
    return [Batch(x) for x in pt.generic_scatter(obj, chunks)]


def dict_gather(batches):
    return pt.generic_gather([b.value for b in batches])


def dict_batch_size(obj):
    return pt.leading_size(obj)


DICT_SG = ScatterGatherFn(scatter=dict_scatter, gather=dict_gather, batch_size=dict_batch_size)


def mask_tokens(ids: torch.Tensor, attn: torch.Tensor, vocab: int, mask_id: int = 3, mlm_p: float = 0.15,
                generator=None):
    """15 % of the real tokens become prediction targets: 80 % -> [MASK], 10 % -> random, 10 % kept."""
    prob = torch.rand(ids.shape, generator=generator)
    pick = (prob < mlm_p) & attn.bool()
    labels = torch.where(pick, ids, torch.full_like(ids, -100))
    r = torch.rand(ids.shape, generator=generator)
    out = ids.clone()
    out[pick & (r < 0.8)] = mask_id
    rnd = pick & (r >= 0.8) & (r < 0.9)
    out[rnd] = torch.randint(1000 if vocab > 2000 else 4, vocab, (int(rnd.sum()),), generator=generator)
    return out, labels


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--teacher", default="bert_base", choices=["bert_base", "bert_large", "tiny"])
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--lr", type=float, default=5e-4)
    ap.add_argument("--warmup-prop", type=float, default=0.05)
    ap.add_argument("--temperature", type=float, default=2.0)
    ap.add_argument("--alpha-ce", type=float, default=5.0)
    ap.add_argument("--alpha-mlm", type=float, default=2.0)
    ap.add_argument("--alpha-cos", type=float, default=1.0)
    ap.add_argument("--artifact-dir", default="runs/distilbert")
    ap.add_argument("--plain", action="store_true", help="the reference's non-pipelined trainer (one device)")
    args, _ = ap.parse_known_args()
    tcfg, scfg = {"bert_base": (B.BERT_BASE, B.DISTILBERT_BASE), "bert_large": (B.BERT_LARGE, B.BertConfig(
        hidden=1024, layers=12, heads=16, ffn=4096, distil=True)), "tiny": (B.BERT_TINY_TEST, B.DISTIL_TINY_TEST)}[args.teacher]
    student, teacher = B.distillation_pair(tcfg, scfg)
    opt = AdamW(student.parameters(), lr=args.lr, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.0)
    extra = Namespace(temperature=args.temperature, alpha_ce=args.alpha_ce, alpha_mlm=args.alpha_mlm,
                      alpha_cos=args.alpha_cos)
    if args.plain:
        tsp = PlainTrainer(student, teacher, None, opt, distil_loss, None, 1.0, args.artifact_dir, supervised=True,
                           target_train_mode=False, scatter_gather_fn=DICT_SG, extra_args=extra)
    else:
        tsp = TSPipe(student, teacher, None, opt, distil_loss, None, 1.0, args.artifact_dir,
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False, scatter_gather_fn=DICT_SG,
                     extra_args=extra)
    g = torch.Generator().manual_seed(0)
    seq = min(args.seq_len, tcfg.max_pos)
    log = RunLog(args.artifact_dir, enabled=tsp.is_primary())      # TensorBoard scalars + scalars.csv + model.pth
    for it in range(args.iters):
        ids = torch.randint(1000 if tcfg.vocab_size > 2000 else 4, tcfg.vocab_size, (args.batch_size, seq), generator=g)
        attn = torch.ones_like(ids)
        masked, labels = mask_tokens(ids, attn, tcfg.vocab_size, mask_id=103 if tcfg.vocab_size > 2000 else 3, generator=g)
        batch = {"input_ids": masked, "attention_mask": attn}
        counts = (int((labels >= 0).sum()), int(attn.sum()))
        tsp.update_lr(linear_warmup_decay(it, args.iters, args.lr, int(args.warmup_prop * args.iters)))
        loss = tsp.feed(batch, batch, (labels, attn) + counts)
        if loss is not None:
            log.scalar("loss", loss, it + 1)
            if (it + 1) % 10 == 0 and tsp.is_primary():
                print(f"iter {it + 1} loss {loss:.4f} {tsp.meter.recent():.1f} samples/s", flush=True)
    for k, loss in enumerate(tsp.stop()):
        log.scalar("loss", loss, args.iters + 1 + k)
    log.scalar("samples_per_second", tsp.meter.overall(), args.iters)
    log.save_final(tsp, opt)
    log.close()


if __name__ == "__main__":
    main()
