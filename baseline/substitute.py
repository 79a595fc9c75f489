"""Substitute reference arm for the workloads whose reference application cannot run on this image.

The reference's MoCo-v3 and soft-target KD applications import ``timm`` (`benchmarks/moco-v3/vits.py:13-15`,
`benchmarks/soft_target/models/vits.py`), its DistilBERT application relies on ``transformers`` 4.x internals
(`benchmarks/distilbert/bert.py:122-130`); neither package (version) is installed and nothing can be downloaded.
What stands in for them is what those applications' own non-pipelined baselines are: the same architectures in
plain PyTorch (``nn.TransformerEncoderLayer`` blocks, library attention / GEMMs, ``torch.optim.AdamW``) trained
with NCCL ``DistributedDataParallel``, one replica per GPU (`benchmarks/moco-v3/main.py:249-254` builds exactly
that; keys all-gathered as in `moco/builder.py:138-149`).  Nothing from ``tspipe_b200`` is imported here.  Every
output line says ``"reference_class": "substitute"``.

    torchrun --nproc-per-node N bench.py --impl reference --workload moco|distilbert|kd --gpus N --steps K --warmup W
"""
from __future__ import annotations

import json
import os
import sys
import time


def _vit(torch, nn, dim, depth, heads, num_classes=0, img=224, patch=16):
    class ViT(nn.Module):
        def __init__(self):
            super().__init__()
            self.patch = nn.Conv2d(3, dim, patch, patch)
            n = (img // patch) ** 2
            self.cls = nn.Parameter(torch.zeros(1, 1, dim))
            self.pos = nn.Parameter(torch.randn(1, n + 1, dim) * 0.02)
            layer = nn.TransformerEncoderLayer(dim, heads, 4 * dim, dropout=0.0, activation="gelu", batch_first=True,
                                               norm_first=True)
            self.blocks = nn.TransformerEncoder(layer, depth, enable_nested_tensor=False)
            self.norm = nn.LayerNorm(dim, eps=1e-6)
            self.head = nn.Linear(dim, num_classes) if num_classes else nn.Identity()

        def forward(self, x):
            x = self.patch(x).flatten(2).transpose(1, 2)
            x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], 1) + self.pos
            return self.head(self.norm(self.blocks(x))[:, 0])
    return ViT()


def _mlp(nn, n_layers, din, dmid, dout, last_bn=True):
    layers = []
    for i in range(n_layers):
        a, b = (din if i == 0 else dmid), (dout if i == n_layers - 1 else dmid)
        layers.append(nn.Linear(a, b, bias=False))
        if i < n_layers - 1:
            layers += [nn.BatchNorm1d(b), nn.ReLU(inplace=True)]
        elif last_bn:
            layers.append(nn.BatchNorm1d(b, affine=False))
    return nn.Sequential(*layers)


def _bert(torch, nn, layers, hidden=768, heads=12, ffn=3072, vocab=30522, max_pos=512):
    class Bert(nn.Module):
        def __init__(self):
            super().__init__()
            self.word, self.posn, self.seg = nn.Embedding(vocab, hidden), nn.Embedding(max_pos, hidden), nn.Embedding(2, hidden)
            self.emb_norm = nn.LayerNorm(hidden, eps=1e-12)
            layer = nn.TransformerEncoderLayer(hidden, heads, ffn, dropout=0.0, activation="gelu", batch_first=True,
                                               norm_first=False)
            self.enc = nn.TransformerEncoder(layer, layers, enable_nested_tensor=False)
            self.dense, self.head_norm = nn.Linear(hidden, hidden), nn.LayerNorm(hidden, eps=1e-12)
            self.bias = nn.Parameter(torch.zeros(vocab))

        def forward(self, ids):
            pos = torch.arange(ids.shape[1], device=ids.device)
            h = self.emb_norm(self.word(ids) + self.posn(pos)[None] + self.seg.weight[0])
            h = self.enc(h)
            z = self.head_norm(torch.nn.functional.gelu(self.dense(h)))
            return torch.nn.functional.linear(z, self.word.weight, self.bias), h
    return Bert()


def run_substitute(a) -> None:
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch import nn
    from torch.nn.parallel import DistributedDataParallel as DDP

    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != a.gpus:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"launched with {world} ranks for --gpus {a.gpus}"}))
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29578")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    per_gpu = a.per_gpu_batch or {"moco": 512, "distilbert": 32, "kd": 256}[a.workload]
    global_batch = per_gpu * world
    w = a.workload

    def build():
        torch.manual_seed(0)
        if w == "moco":
            enc = nn.Sequential(_vit(torch, nn, 768, 12, 12), _mlp(nn, 3, 768, 4096, 256)).to(dev)
            mom = nn.Sequential(_vit(torch, nn, 768, 12, 12), _mlp(nn, 3, 768, 4096, 256)).to(dev)
            pred = _mlp(nn, 2, 256, 4096, 256).to(dev)
            for p in mom.parameters():
                p.requires_grad_(False)
            student = nn.Sequential(enc, pred)
            return student, mom, torch.optim.AdamW(student.parameters(), lr=1.5e-4 * global_batch / 256, weight_decay=0.1,
                                                   fused=True)
        if w == "kd":
            student, teacher = _vit(torch, nn, 768, 12, 12, 1000).to(dev), _vit(torch, nn, 1024, 24, 16, 1000).to(dev).eval()
            for p in teacher.parameters():
                p.requires_grad_(False)
            return student, teacher, torch.optim.AdamW(student.parameters(), lr=1e-3, weight_decay=0.05, fused=True)
        student, teacher = _bert(torch, nn, 6).to(dev), _bert(torch, nn, 12).to(dev).eval()
        for p in teacher.parameters():
            p.requires_grad_(False)
        return student, teacher, torch.optim.AdamW(student.parameters(), lr=5e-4, betas=(0.9, 0.98), eps=1e-6,
                                                   weight_decay=0.0, fused=True)

    def gather(k):
        if world == 1:
            return k
        out = [torch.empty_like(k) for _ in range(world)]
        dist.all_gather(out, k)
        return torch.cat(out)

    def nce(q, k, T=0.2):
        q, k = F.normalize(q.float(), dim=1), gather(F.normalize(k.float(), dim=1))
        logits = q @ k.t() / T
        labels = torch.arange(q.shape[0], device=dev) + q.shape[0] * rank
        return F.cross_entropy(logits, labels) * 2 * T

    def make_batch(g):
        if w == "distilbert":
            ids = torch.randint(1000, 30522, (per_gpu, a.seq_len), generator=g)
            pick = torch.rand(ids.shape, generator=g) < 0.15
            labels = torch.where(pick, ids, torch.full_like(ids, -100))
            r = torch.rand(ids.shape, generator=g)
            masked = ids.clone()
            masked[pick & (r < 0.8)] = 103
            rnd = pick & (r >= 0.8) & (r < 0.9)
            masked[rnd] = torch.randint(1000, 30522, (int(rnd.sum()),), generator=g)
            return (masked.pin_memory(), labels.pin_memory())
        x1 = torch.randn(per_gpu, 3, a.image, a.image, generator=g).pin_memory()
        if w == "moco":
            return (x1, torch.randn(per_gpu, 3, a.image, a.image, generator=g).pin_memory())
        return (x1, torch.randint(0, 1000, (per_gpu,), generator=g).pin_memory())

    def run(dtype: str):
        student, teacher, opt = build()
        ddp = DDP(student, device_ids=[local]) if world > 1 else student
        amp = torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == "bf16")
        g = torch.Generator().manual_seed(1234 + rank)
        host = [make_batch(g) for _ in range(2)]
        devb = [tuple(t.to(dev) for t in b) for b in host]

        def step(b):
            with amp:
                if w == "moco":
                    x1, x2 = b
                    q1, q2 = ddp(x1), ddp(x2)
                    with torch.no_grad():
                        for ps, pt_ in zip(student[0].parameters(), teacher.parameters()):
                            pt_.mul_(0.99).add_(ps.detach(), alpha=0.01)
                        k1, k2 = teacher(x1), teacher(x2)
                    loss = nce(q1, k2) + nce(q2, k1)
                elif w == "kd":
                    x, y = b
                    s = ddp(x)
                    with torch.no_grad():
                        t = teacher(x)
                    loss = F.cross_entropy(s.float(), y) + 16.0 * F.kl_div(F.log_softmax(s.float() / 4, 1),
                                                                            F.softmax(t.float() / 4, 1), reduction="batchmean")
                else:
                    ids, labels = b
                    s_logits, s_h = ddp(ids)
                    with torch.no_grad():
                        t_logits, t_h = teacher(ids)
                    v = s_logits.shape[-1]
                    sl, tl = s_logits.float().view(-1, v), t_logits.float().view(-1, v)
                    loss = 5.0 * 4.0 * F.kl_div(F.log_softmax(sl / 2, -1), F.softmax(tl / 2, -1), reduction="batchmean") \
                        + 2.0 * F.cross_entropy(sl, labels.view(-1), ignore_index=-100)
                    hs, ht = s_h.float().view(-1, s_h.shape[-1]), t_h.float().view(-1, t_h.shape[-1])
                    loss = loss + F.cosine_embedding_loss(hs, ht, torch.ones(hs.shape[0], device=dev))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            return loss

        def timed(steps, from_host):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            last = None
            for i in range(steps):
                b = tuple(t.to(dev, non_blocking=True) for t in host[i % 2]) if from_host else devb[i % 2]
                loss = step(b)
                if from_host:
                    last = float(loss)           # the loss goes back to the host every step
            e1.record()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) * 1e3
            t = torch.tensor([e0.elapsed_time(e1), wall], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t[0].item(), t[1].item(), (last if from_host else float(loss))

        for i in range(a.warmup):
            step(devb[i % 2])
        ms, _, last = timed(a.steps, False)
        ms2, wall2, _ = timed(a.steps, True)
        in_bytes = sum(t.numel() * t.element_size() for t in host[0]) * world
        res = {"value": round(global_batch * a.steps / (ms / 1e3), 2), "ms_per_step": round(ms / a.steps, 3),
               "last_loss": round(last, 5),
               "e2e": {"value": round(global_batch * a.steps / (max(ms2, wall2) / 1e3), 2), "ms_per_step":
                       round(max(ms2, wall2) / a.steps, 3), "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": 4 * world}}
        del student, teacher, opt, ddp, devb
        torch.cuda.empty_cache()
        return res

    metric = {"moco": "MoCo-v3 ViT-B/16 training throughput", "distilbert": "DistilBERT-style KD training throughput",
              "kd": "Soft-target KD ViT-L/16 -> ViT-B/16 training throughput"}[w]
    unit = "images/s" if w == "moco" else "samples/s"
    want = getattr(a, "ref_dtype", "auto")
    if want == "auto":
        want = "both"
    try:
        main = run("fp32" if want == "fp32" else "bf16")
        extra = run("fp32") if want == "both" else None
    except Exception as e:  # noqa: BLE001 - reported in the output line
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"substitute run failed: {e!r}"[:300]}), flush=True)
        dist.destroy_process_group()
        return
    if rank == 0:
        out = {"metric": metric, "value": main["value"], "unit": unit, "n_gpus": world, "steps": a.steps,
               "warmup": a.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": "fp32 (TF32 tensor cores)" if want == "fp32" else "bf16 (torch.autocast)",
               "data": "synthetic", "impl": "reference", "reference_class": "substitute",
               "why_substitute": "the reference application needs timm / transformers 4.x, which the image lacks; this is "
                                 "the same architecture in plain PyTorch + NCCL DistributedDataParallel",
               "config": {"model": {"moco": "mocov3_vit_base+mlp4096-256", "distilbert": "bert12L->distilbert6L seq512",
                                    "kd": "vit_large->vit_base"}[w], "global_batch": global_batch,
                          "seq_len": a.seq_len if w == "distilbert" else None, "image": a.image if w != "distilbert" else None,
                          "parallelism": f"ddp{world}", "microbatches": 1, "bwd_split": 1, "optimizer": "AdamW (fused)",
                          "ema": 0.99 if w == "moco" else None, "views": "one forward per view",
                          "l2_policy": "inputs larger than L2 (a step's activations are several GB per GPU)",
                          "timing": "CUDA events around K steps, max over ranks"},
               "last_loss": main["last_loss"], "e2e": dict(main["e2e"], unit=unit,
                                                            api="pinned host batch -> device, step, float(loss) every step")}
        if extra is not None:
            out["reference_fp32"] = {"value": extra["value"], "unit": unit, "ms_per_step": extra["ms_per_step"],
                                     "dtype": "fp32 (TF32 tensor cores)"}
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    run_substitute(bench.parse())
