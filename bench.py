#!/usr/bin/env python
"""Training-throughput benchmarks on N B200 GPUs of one node.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload byol|moco|distilbert|kd]

For N > 1 the script is launched once per GPU (``python -m torch.distributed.run --nproc-per-node N
... bench.py --gpus N ...``); started plainly with ``--gpus N > 1`` it re-launches itself that way.

Workloads (synthetic N(0,1) / uniform-token inputs, random-init weights, bf16 compute with fp32 master
parameters, weak scaling: the per-GPU batch is fixed as N grows):

``byol`` (default, the headline)  BYOL, ResNet-50 trunks + 2048-4096-256 projector (+ 256-4096-256 predictor on the
    online net), two 224x224x3 views per sample, LARS, target EMA 0.996; 128 samples per GPU (global batch 1024 at
    8 GPUs).
``moco``   MoCo-v3, ViT-B/16 encoders + 3-layer projector (+ 2-layer predictor), InfoNCE T = 0.2 over the keys of all
    replicas, AdamW, momentum 0.99; 512 samples per GPU (global batch 4096 at 8 GPUs).
``distilbert``  BERT-12L teacher (frozen) -> 6-layer student, sequence length 512, MLM masking 15 % (80/10/10), loss
    5.0 * soft CE at T = 2 + 2.0 * MLM CE + 1.0 * hidden-state cosine, AdamW; 32 sequences per GPU (256 at 8 GPUs).
``kd``     soft-target KD, ViT-L/16 teacher (frozen) -> ViT-B/16 student, CE + KL at T = 4, AdamW; 256 samples per GPU
    (2048 at 8 GPUs).  From 2 GPUs on the default grid is split placement: teacher stages on the first half of the
    ranks, student stages on the second half (4 + 4 at 8 GPUs, 16 microbatches), the KD loss reading the teacher
    logits from the teacher GPU's memory.

Own arm (``tspipe_b200``): ranks form a ``dp x pp`` grid, each pipeline runs the interleaved teacher/student schedule
with delayed EMA.  Two timed passes of exactly K steps, each bracketed by barrier + synchronize, timed with CUDA
events on the compute stream, max over ranks: ``value`` feeds device-resident inputs; ``e2e`` goes through
``TSPipe.feed`` with pinned host inputs (H2D every step) and reads every step's loss back (D2H).  A pass ends with
``TSPipe.flush`` so it contains the complete work of its K steps including pipeline fill and drain.  ``pipeline``
lists the same job on the pipelined grids that fit N (``ppN``, ``dp(N/2) x pp2``, ``dp(N/4) x pp4``) with the per-
operation device-time totals of each.

Reference arm (``--impl reference``): ``byol`` runs the unmodified reference package from ``baseline/_ref`` through
its own ``TSPipe`` API (``baseline/run_reference.py``); the other workloads need packages the image does not have
(``timm``, ``transformers`` 4.x), so their reference arm is a stated substitute: the same architectures in plain
PyTorch + NCCL DistributedDataParallel (``baseline/substitute.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

BASELINE_PUBLISHED = None     # the reference publishes no absolute throughput

WORKLOADS = {
    #             metric                                            unit         per-GPU batch  model tag
    "byol": ("BYOL ResNet-50 training throughput", "images/s", 128, "byol_resnet50+mlp4096-256"),
    "moco": ("MoCo-v3 ViT-B/16 training throughput", "images/s", 512, "mocov3_vit_base+mlp4096-256"),
    "distilbert": ("DistilBERT-style KD training throughput", "samples/s", 32, "bert12L->distilbert6L seq512"),
    "kd": ("Soft-target KD ViT-L/16 -> ViT-B/16 training throughput", "samples/s", 256, "vit_large->vit_base"),
}


def parse(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="byol", choices=sorted(WORKLOADS))
    p.add_argument("--pp", type=int, default=0, help="pipeline stages (0 = default for this GPU count)")
    p.add_argument("--ubatch", type=int, default=0, help="forward microbatches (0 = default)")
    p.add_argument("--bwd-split", type=int, default=0)
    p.add_argument("--per-gpu-batch", type=int, default=0, help="0 = the workload's default")
    p.add_argument("--model", default="resnet50")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"], help="compute dtype (fp32 = TF32 tensor cores)")
    p.add_argument("--host-dtype", default="bf16", choices=["bf16", "fp32"],
                   help="dtype of the pinned host inputs of the end-to-end pass (image workloads)")
    p.add_argument("--ref-dtype", default="auto", choices=["auto", "fp32", "bf16", "both"],
                   help="reference arm: as shipped (fp32), under bf16 autocast, or both")
    p.add_argument("--no-fused", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--pipeline-budget", type=int, default=300,
                   help="seconds the secondary pipelined grids may take before the headline is printed without them")
    p.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false",
                   help="run every stage eagerly instead of replaying stage forwards / backwards from CUDA graphs")
    p.add_argument("--cuda-graphs", dest="cuda_graphs", action="store_true", help=argparse.SUPPRESS)
    p.set_defaults(cuda_graphs=True)
    p.add_argument("--no-pipeline", action="store_true", help="skip the secondary pipelined-grid measurements")
    p.add_argument("--image", type=int, default=224)
    p.add_argument("--seq-len", type=int, default=512)
    p.add_argument("--split", default="", help="override model_split, e.g. 9,21/9,17 (online/target)")
    p.add_argument("--placement", default="", choices=["", "colocated", "split"])
    p.add_argument("--trace", action="store_true", help="print per-operation device time totals of the timed pass")
    p.add_argument("--no-peer", action="store_true", help="NCCL all-reduce instead of the peer-memory DP kernels")
    p.add_argument("--sm-reserve", type=int, default=-1, help="SMs left free of the persistent kernels (-1 = default)")
    p.add_argument("--no-merge-views", action="store_true", help="one forward per view instead of stacked views")
    p.add_argument("--no-dp-signals", action="store_true", help="order the DP kernels with NCCL collectives")
    p.add_argument("--no-dp-early", action="store_true", help="reduce the gradients at the optimizer step only")
    p.add_argument("--conv", choices=["igemm", "library"], default=None,
                   help="1x1 / 3x3 convolutions on the tcgen05 implicit-GEMM kernels (default) or the library's")
    p.add_argument("--linear", choices=["tcgen05", "library"], default=None,
                   help="linear layers on the tcgen05 GEMM kernels (default) or the library's")
    return p.parse_args(argv)


# -------------------------------------------------------------------------------------------------
class ClockSampler:
    """``nvidia-smi`` clocks / throttle reasons sampled every 200 ms while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm = sorted(int(float(r[1])) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [int(float(r[2])) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for nme, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ResNet-50 online net = 26 trunk+projector children + 4 predictor children; target = 26.
# Cuts of the 30 student / 26 teacher children (stem = 4 children, 16 residual blocks, pool, reshape, 4 head layers,
# 4 predictor layers), teacher and student cut alike so that the momentum update stays local.  The front of the
# network is the expensive part at 224 x 224: measured forward times per stacked microbatch of 256 samples are 1.28 ms
# for the stem, 0.63 ms per layer1 block, 1.05 ms for the first layer2 block and 4.0 ms for everything behind it, so
# the 4- and 8-stage cuts give the stem a stage (almost) of its own.
BYOL_SPLITS = {
    1: ([30], [26]),
    2: ([8, 22], [8, 18]),
    4: ([5, 3, 6, 16], [5, 3, 6, 12]),
    8: ([4, 2, 1, 1, 3, 3, 4, 12], [4, 2, 1, 1, 3, 3, 4, 8]),
}


def _balance(n_children: int, parts: int):
    from tspipe_b200.tspipe import default_balance
    return default_balance(n_children, parts)


def build_workload(a, world: int, pp: int, placement: str):
    """Models, optimizer, loss and input factory of ``a.workload``; returns a dict."""
    import torch
    from argparse import Namespace
    from tspipe_b200 import TSPipeMode, defaultScatterGatherFn
    from tspipe_b200.losses import byol_loss, distil_loss, ema_update, moco_loss, soft_target_kd
    from tspipe_b200.optim import LARS, AdamW
    w = a.workload
    per_gpu = a.per_gpu_batch or WORKLOADS[w][2]
    global_batch = per_gpu * world
    img = (3, a.image, a.image)
    out = {"global_batch": global_batch, "per_gpu": per_gpu, "mode": TSPipeMode.SELF_SUPERVISED_MOMENTUM,
           "target_train_mode": True, "extra_args": Namespace(), "sg": defaultScatterGatherFn, "predictor": None,
           "update_fn": ema_update, "seq_len": None, "deferred_bn": True}
    torch.manual_seed(0)
    if w == "byol":
        from tspipe_b200.models.resnet import byol_networks
        online, target, predictor = byol_networks(a.model, 4096, 256)
        params = list(online.parameters()) + list(predictor.parameters())
        out.update(online=online, target=target, predictor=predictor, momentum=0.996, loss_fn=byol_loss,
                   opt=LARS(params, lr=0.2 * global_batch / 256, weight_decay=1.5e-6, momentum=0.9),
                   optimizer="LARS", splits=BYOL_SPLITS.get(pp) if a.model == "resnet50" else None)

        def make(batch, gen, dtype):
            return [torch.randn((batch,) + img, generator=gen).to(dtype) for _ in range(2)], None
    elif w == "moco":
        from tspipe_b200.models.vit import moco_vit_networks
        online, target, predictor = moco_vit_networks("vit_base", 256, 4096)
        params = list(online.parameters()) + list(predictor.parameters())
        out.update(online=online, target=target, predictor=predictor, momentum=0.99, loss_fn=moco_loss,
                   opt=AdamW(params, lr=1.5e-4 * global_batch / 256, weight_decay=0.1), optimizer="AdamW",
                   extra_args=Namespace(moco_t=0.2), splits=None)

        def make(batch, gen, dtype):
            return [torch.randn((batch,) + img, generator=gen).to(dtype) for _ in range(2)], None
    elif w == "kd":
        from tspipe_b200.models.vit import vit_classifier
        student, teacher = vit_classifier("vit_base", 1000), vit_classifier("vit_large", 1000)
        out.update(online=student, target=teacher, momentum=1.0, loss_fn=soft_target_kd, update_fn=None,
                   opt=AdamW(student.parameters(), lr=1e-3, weight_decay=0.05), optimizer="AdamW",
                   mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False, deferred_bn=False,
                   extra_args=Namespace(T=4.0, lambda_kd=1.0), splits=None)

        def make(batch, gen, dtype):
            x = torch.randn((batch,) + img, generator=gen).to(dtype)
            return [x, x], torch.randint(0, 1000, (batch,), generator=gen)
    else:
        sys.path.insert(0, os.path.join(REPO, "benchmarks", "distilbert"))
        import train as distil_app          # dict scatter/gather and the MLM masking of the application
        from tspipe_b200.models import bert as B
        student, teacher = B.distillation_pair(B.BERT_BASE, B.DISTILBERT_BASE)
        out.update(online=student, target=teacher, momentum=1.0, loss_fn=distil_loss, update_fn=None,
                   opt=AdamW(student.parameters(), lr=5e-4, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.0),
                   optimizer="AdamW", mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False, deferred_bn=False,
                   sg=distil_app.DICT_SG, seq_len=a.seq_len, splits=None,
                   extra_args=Namespace(temperature=2.0, alpha_ce=5.0, alpha_mlm=2.0, alpha_cos=1.0))
        vocab = B.BERT_BASE.vocab_size

        def make(batch, gen, dtype):
            ids = torch.randint(1000, vocab, (batch, a.seq_len), generator=gen)
            attn = torch.ones_like(ids)
            masked, labels = distil_app.mask_tokens(ids, attn, vocab, mask_id=103, generator=gen)
            b = {"input_ids": masked, "attention_mask": attn}
            return [b, b], (labels, attn, int((labels >= 0).sum()), int(attn.sum()))
    out["make"] = make
    n_on = len(out["online"]) + (len(out["predictor"]) if out["predictor"] is not None else 0)
    n_tg = len(out["target"])
    if placement == "split":
        half = world // 2
        out["splits"] = (_balance(n_on, half), _balance(n_tg, half))
    elif out.get("splits") is None:
        out["splits"] = (_balance(n_on, pp), _balance(n_tg, pp))
    return out


def _pin(obj):
    import torch
    from tspipe_b200.utils import pytree as pt
    if isinstance(obj, (tuple, list)):
        return type(obj)(_pin(o) for o in obj)
    if isinstance(obj, dict) or isinstance(obj, torch.Tensor):
        return pt.tree_map_tensors(lambda t: t.pin_memory(), obj)
    return obj


def _to_dev(obj, dev):
    import torch
    from tspipe_b200.utils import pytree as pt
    if isinstance(obj, (tuple, list)):
        return type(obj)(_to_dev(o, dev) for o in obj)
    if isinstance(obj, dict) or isinstance(obj, torch.Tensor):
        return pt.tree_map_tensors(lambda t: t.to(dev), obj)
    return obj


def _nbytes(obj) -> int:
    import torch
    if isinstance(obj, torch.Tensor):
        return obj.numel() * obj.element_size()
    if isinstance(obj, dict):
        return sum(_nbytes(v) for v in obj.values())
    if isinstance(obj, (tuple, list)):
        return sum(_nbytes(v) for v in obj)
    return 0


def measure(a, pp, dp, ub, split, e2e, placement="colocated"):
    """Build the job on a ``dp x pp`` grid (or a split teacher / student placement), warm up, time K steps."""
    import gc
    import torch
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.ops import fused

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    wl = build_workload(a, world, pp, placement)
    on_split, tg_split = wl["splits"]
    if a.split and pp > 1:
        on_split, tg_split = ([int(x) for x in part.split(",")] for part in a.split.split("/"))
    cfg = {"model_split": {"online": on_split, "target": tg_split},
           "runtime": {"num_ubatch": ub, "bwd_split": split, "dp_replicas": dp, "dtype": a.dtype,
                       "fused": not a.no_fused, "channels_last": True, "max_inflight": 3, "timeout_s": 120,
                       "peer_memory": not a.no_peer, "cuda_graphs": a.cuda_graphs, "placement": placement,
                       "dp_signals": not a.no_dp_signals, "dp_early_reduce": not a.no_dp_early,
                       "merge_views": not a.no_merge_views, "sm_reserve": None if a.sm_reserve < 0 else a.sm_reserve},
           "train": {"deferred_batch_norm": wl["deferred_bn"]}}
    from tspipe_b200.profiler import TSPipeProfiler
    prof = TSPipeProfiler(filename=f"/tmp/bench_trace_{rank}.csv").__enter__()
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(wl["online"], wl["target"], wl["predictor"], wl["opt"], wl["loss_fn"], wl["update_fn"],
                     wl["momentum"], "", tspipe_mode=wl["mode"], target_train_mode=wl["target_train_mode"],
                     extra_args=wl["extra_args"], scatter_gather_fn=wl["sg"], config=cfg, device=dev, profiler=prof)
    topo = tsp.topo
    global_batch = wl["global_batch"]
    replica_batch = global_batch // dp
    g = torch.Generator().manual_seed(1234 + topo.replica)
    n_host = 2
    host_dtype = torch.bfloat16 if (a.host_dtype == "bf16" and a.dtype == "bf16") else torch.float32
    feeds_inputs = bool(topo.is_first)
    feeds_labels = bool(getattr(topo, "is_loss_rank", topo.is_last)) and wl["mode"].name.startswith("SUPERVISED")
    host_sets = dev_sets = None
    in_bytes = 0
    if feeds_inputs or feeds_labels:
        host_sets, dev_sets = [], []
        for _ in range(n_host):
            views, labels = wl["make"](replica_batch, g, host_dtype)
            views = views if feeds_inputs else [None, None]
            labels = labels if (feeds_labels or feeds_inputs) else None
            hv = [_pin(v) if v is not None else None for v in ([views[0]] if views[0] is views[1] else views)]
            if len(hv) == 1:
                hv = [hv[0], hv[0]]
            hl = _pin(labels) if labels is not None else None
            host_sets.append((hv, hl))
            dv0 = _to_dev(hv[0], dev) if hv[0] is not None else None
            dv = [dv0, dv0 if hv[1] is hv[0] else (_to_dev(hv[1], dev) if hv[1] is not None else None)]
            dev_sets.append((dv, hl))
        hv, hl = host_sets[0]
        in_bytes = (_nbytes(hv[0]) + (0 if hv[1] is hv[0] else _nbytes(hv[1])) if feeds_inputs else 0) + _nbytes(hl)

    supervised = wl["mode"].name.startswith("SUPERVISED")

    def feed(i, host):
        if host_sets is None:            # a rank that holds neither a first stage nor the loss stage feeds nothing
            return tsp.feed(None, None, 0) if supervised else tsp.feed(None, None)
        views, labels = (host_sets if host else dev_sets)[i % n_host]
        if supervised:
            return tsp.feed(views[0], views[1], labels if labels is not None else 0)
        return tsp.feed(views[0], views[1])

    def timed(steps, host, sampler=None):
        dist.barrier()
        torch.cuda.synchronize()
        l0 = fused.LAUNCHES
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.start()
        e0.record(tsp.engine.compute)
        t0 = time.perf_counter()
        losses = []
        for i in range(steps):
            l = feed(i, host)
            if l is not None:
                losses.append(l)
        losses += tsp.flush()
        e1.record(tsp.engine.compute)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        clocks = sampler.stop() if sampler else None
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms, wall * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        n_launch = torch.tensor([fused.LAUNCHES - l0], device=dev)
        dist.all_reduce(n_launch)
        return t[0].item(), t[1].item(), losses, clocks, int(n_launch.item())

    for i in range(a.warmup):          # untimed warm-up
        feed(i, False)
    tsp.flush()
    prof.device_events.clear()
    ms, wall_ms, losses, clocks, launches = timed(a.steps, False, ClockSampler(local) if rank == 0 else None)
    tot = {}
    for op, row, dms in prof.device_times():
        tot[op] = tot.get(op, 0.0) + dms
    trace = {k: round(v / a.steps, 3) for k, v in sorted(tot.items())}
    if a.trace:
        print(f"[trace rank {rank} stage {topo.stage} replica {topo.replica}] per-step device ms: " +
              ", ".join(f"{k}={v:.2f}" for k, v in trace.items()), flush=True)
    prof.device_events.clear()
    # the slowest rank's per-operation totals describe the critical path
    gathered = [None] * world
    dist.all_gather_object(gathered, (rank, int(topo.stage), int(topo.replica), bool(getattr(topo, "is_teacher", False)),
                                      trace))
    out = {"value": round(global_batch * a.steps / (ms / 1e3), 2), "ms_per_step": round(ms / a.steps, 3),
           "gpu_launches": launches, "clocks": clocks, "microbatches": ub,
           "parallelism": (f"split placement: {pp} teacher stages + {pp} student stages, dp{dp}"
                           if placement == "split" else f"dp{dp}xpp{pp}"),
           "bwd_split": split, "global_batch": global_batch, "merged_views": bool(getattr(tsp.engine, "merge_views", False)),
           "last_loss": round(losses[-1], 5) if losses else None, "optimizer": wl["optimizer"], "seq_len": wl["seq_len"],
           # per-operation device time of replica 0's stages (compute = forwards, backward, loss, optimize)
           "device_ms_per_step_by_op": {("teacher" if tch else "") + f"stage{s}": t
                                        for r, s, rep, tch, t in sorted(gathered, key=lambda x: x[0]) if rep == 0}}
    if e2e:
        for i in range(min(a.warmup, 3)):
            feed(i, True)
        tsp.flush()
        ms2, wall2, losses2, _, _ = timed(a.steps, True)
        out["e2e"] = {"value": round(global_batch * a.steps / (max(ms2, wall2) / 1e3), 2), "unit": WORKLOADS[a.workload][1],
                      "h2d_bytes_per_step": int(_sum_over_ranks(in_bytes, dev)), "d2h_bytes_per_step": 4 * dp,
                      "ms_per_step": round(max(ms2, wall2) / a.steps, 3), "host_input_dtype": str(host_dtype).replace("torch.", ""),
                      "api": "TSPipe.feed(pinned host inputs) per step; loss read back per step; TSPipe.flush at the end"}
    tsp.stop()
    prof.__exit__(None, None, None)
    del tsp, wl, host_sets, dev_sets
    gc.collect()
    torch.cuda.empty_cache()
    return out


def _sum_over_ranks(v, dev):
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(v)], device=dev, dtype=torch.float64)
    dist.all_reduce(t)
    return t.item()


def pipeline_grids(world: int, workload: str):
    """Pipelined grids measured next to the headline: (pp, dp, microbatches)."""
    if workload != "byol":
        return []
    grids = []
    if world >= 2:
        grids.append((world, 1, world))              # one pipeline over all GPUs, N microbatches
    if world >= 4:
        grids.append((2, world // 2, 2))
    if world >= 8:
        grids.append((4, world // 4, 4))
    return grids


def run_ours(a):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    assert world == a.gpus, f"launched with {world} ranks for --gpus {a.gpus}"
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    os.environ.setdefault("TORCH_NCCL_SHOW_EAGER_INIT_P2P_SERIALIZATION_WARNING", "false")
    torch.cuda.set_device(local)
    torch.backends.cudnn.benchmark = True
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True

    if a.conv is not None:
        from tspipe_b200.ops import conv as _conv
        _conv.set_igemm(a.conv == "igemm")
    if a.linear is not None:
        from tspipe_b200.ops import linear as _linear
        _linear.set_tcgen05(a.linear == "tcgen05")
    metric, unit, _, model = WORKLOADS[a.workload]
    # Default grid: every GPU holds a whole teacher + student replica (models of these sizes are far below one
    # B200's memory); gradients go through the peer-memory reduce-scatter + step + all-gather.  `kd` from 2 GPUs on:
    # split placement, teacher stages and student stages on different GPUs.
    placement = a.placement or ("split" if (a.workload == "kd" and world >= 2 and not a.pp) else "colocated")
    pp, dp, ub, split = 1, world, 1, 1
    if placement == "split":
        pp, dp, ub = world // 2, 1, max(2 * (world // 2), 2)
    if a.pp:
        pp, dp = a.pp, world // a.pp
        ub = max(pp - 1, 1) if pp > 2 else 1
    ub = a.ubatch or ub
    split = a.bwd_split or split
    r = measure(a, pp, dp, ub, split, e2e=not a.no_e2e, placement=placement)
    if a.workload == "byol" and a.model != "resnet50":
        model = f"byol_{a.model}+mlp4096-256"
    out = {"metric": metric, "value": r["value"], "unit": unit,
           "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": r["ms_per_step"],
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": a.dtype if a.dtype == "bf16" else "fp32 (TF32 tensor cores)", "data": "synthetic",
           "impl": "ours", "gpu_launches": r["gpu_launches"], "clocks": r["clocks"],
           "config": {"model": model, "global_batch": r["global_batch"], "seq_len": r["seq_len"],
                      "image": a.image if a.workload != "distilbert" else None, "parallelism": r["parallelism"],
                      "microbatches": r["microbatches"], "bwd_split": r["bwd_split"], "optimizer": r["optimizer"],
                      "ema": {"byol": 0.996, "moco": 0.99}.get(a.workload),
                      "views": "both views of a network in one stacked forward, BatchNorm statistics per view"
                               if r.get("merged_views") else "one forward per view",
                      "l2_policy": "inputs larger than L2 (a step's activations are several GB per GPU)",
                      "timing": "CUDA events on the compute stream around K feeds + flush, max over ranks"},
           "device_ms_per_step_by_op": r["device_ms_per_step_by_op"]}
    if r.get("last_loss") is not None:
        out["last_loss"] = r["last_loss"]
    if "e2e" in r:
        out["e2e"] = r["e2e"]
    guard = None
    if placement == "colocated" and pp == 1 and not a.no_pipeline:
        # the same job on the pipelined grids that fit this GPU count.  They are secondary: if one of them should
        # stall (a rank that failed while the others wait for it), the headline measured above is printed without
        # them when the time budget runs out, and every rank leaves.
        import threading
        printed = threading.Lock()

        def give_up():
            if printed.acquire(blocking=False):
                if rank == 0:
                    out["pipeline_error"] = f"the pipelined grids did not finish within {a.pipeline_budget} s"
                    print(json.dumps(out), flush=True)
                os._exit(0)
        guard = threading.Timer(float(a.pipeline_budget) + (0.0 if rank == 0 else 5.0), give_up)
        guard.daemon = True
        guard.start()
        plist = []
        for gpp, gdp, gub in pipeline_grids(world, a.workload):
            try:
                p2 = measure(a, gpp, gdp, gub, split, e2e=False)
                plist.append({k: p2[k] for k in ("value", "ms_per_step", "parallelism", "microbatches",
                                                 "gpu_launches", "device_ms_per_step_by_op")})
            except Exception as e:  # noqa: BLE001 - the headline above stands on its own
                plist.append({"parallelism": f"dp{gdp}xpp{gpp}", "microbatches": gub,
                              "error": f"{type(e).__name__}: {e}"[:300]})
                break
        if plist:
            out["pipeline"] = plist
        guard.cancel()
        if not printed.acquire(blocking=False):
            return                              # the budget ran out a moment ago: the line is already out
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        import threading
        last = threading.Timer(60.0, lambda: os._exit(0))      # the line is out: never hang in the tear-down
        last.daemon = True
        last.start()
        dist.barrier()
        dist.destroy_process_group()


def relaunch(a):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 400), os.path.abspath(__file__)]
    cmd += sys.argv[1:]
    sys.exit(subprocess.call(cmd))


def main():
    a = parse()
    if a.impl == "reference":
        sys.path.insert(0, os.path.join(REPO, "baseline"))
        if a.workload == "byol":
            from run_reference import run_reference
            return run_reference(a)
        if a.gpus > 1 and "RANK" not in os.environ:
            return relaunch(a)
        from substitute import run_substitute
        return run_substitute(a)
    if a.gpus > 1 and "RANK" not in os.environ:
        return relaunch(a)
    run_ours(a)


if __name__ == "__main__":
    main()
