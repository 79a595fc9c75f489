#!/usr/bin/env python
"""Headline benchmark: BYOL ResNet-50 training throughput (images/s) on N B200 GPUs of one node.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

For N > 1 the script is launched once per GPU (``python -m torch.distributed.run --nproc-per-node N
... bench.py --gpus N ...``); started plainly with ``--gpus N > 1`` it re-launches itself that way.

Workload (both arms): BYOL, ResNet-50 trunks + 2048-4096-256 projector (+ 256-4096-256 predictor on
the online net), two 224x224x3 fp32 views per sample, LARS, target EMA 0.996, bf16 compute,
synthetic N(0,1) inputs, random-init weights.  Weak scaling: 128 samples per GPU per step
(global batch 1024 at 8 GPUs).

Own arm (``tspipe_b200``): ranks form a ``dp x pp`` grid, each pipeline runs the interleaved
teacher/student schedule with delayed EMA.  Two timed passes of exactly K steps, each bracketed by
barrier + synchronize, timed with CUDA events on the compute stream, max over ranks:
``value`` feeds device-resident inputs; ``e2e`` goes through ``TSPipe.feed`` with pinned host inputs
(H2D every step) and reads every step's loss back (D2H).  A pass ends with ``TSPipe.flush`` so it
contains the complete work of its K steps including pipeline fill and drain.

Reference arm: the unmodified reference package from ``baseline/_ref`` driven through its own
``TSPipe`` API (see ``baseline/run_reference.py``).
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

PER_GPU_BATCH = 128
BASELINE_PUBLISHED = None     # the reference publishes no absolute throughput


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--pp", type=int, default=0, help="pipeline stages (0 = default for this GPU count)")
    p.add_argument("--ubatch", type=int, default=0, help="forward microbatches (0 = default)")
    p.add_argument("--bwd-split", type=int, default=0)
    p.add_argument("--per-gpu-batch", type=int, default=PER_GPU_BATCH)
    p.add_argument("--model", default="resnet50")
    p.add_argument("--no-fused", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--cuda-graphs", action="store_true", help="replay teacher stage forwards from CUDA graphs")
    p.add_argument("--no-pipeline", action="store_true", help="skip the secondary two-stage pipeline measurement")
    p.add_argument("--image", type=int, default=224)
    p.add_argument("--split", default="", help="override model_split, e.g. 9,21/9,17 (online/target)")
    p.add_argument("--trace", action="store_true", help="print per-operation device time totals of the timed pass")
    p.add_argument("--no-peer", action="store_true", help="NCCL all-reduce instead of the peer-memory DP kernels")
    p.add_argument("--conv", choices=["igemm", "library"], default=None,
                   help="1x1 / 3x3 convolutions on the tcgen05 implicit-GEMM kernels (default) or the library's")
    return p.parse_args()


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


def default_grid(n: int):
    """(pp, dp, ubatch, bwd_split) per GPU count.  ResNet-50 (33 M parameters) is far below one B200's
    memory, so the headline number replicates the single-stage teacher/student step on every GPU (gradient
    reduce-scatter + LARS + all-gather through peer memory); the interleaved two-stage pipeline on the same
    job is measured next to it (``pipeline`` in the output, ``--pp 2`` to make it the main number)."""
    return 1, n, 1, 1


# ResNet-50 online net = 26 trunk+projector children + 4 predictor children; target = 26.
SPLITS = {
    1: ([30], [26]),
    2: ([8, 22], [8, 18]),
    4: ([6, 5, 7, 12], [6, 5, 7, 8]),
    8: ([5, 2, 3, 3, 3, 3, 4, 7], [5, 2, 3, 3, 3, 3, 4, 3]),
}


def measure(a, pp, dp, ub, split, e2e):
    """Build the BYOL ResNet-50 job on a ``dp x pp`` grid, warm up, time K steps; returns a result dict."""
    import gc
    import torch
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.models.resnet import byol_networks
    from tspipe_b200.optim import LARS
    from tspipe_b200.ops import fused

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    online, target, predictor = byol_networks(a.model, 4096, 256)
    params = list(online.parameters()) + list(predictor.parameters())
    global_batch = a.per_gpu_batch * world
    lr = 0.2 * global_batch / 256
    opt = LARS(params, lr=lr, weight_decay=1.5e-6, momentum=0.9)
    on_split, tg_split = SPLITS[pp]
    if a.split and pp > 1:
        on_split, tg_split = ([int(x) for x in part.split(",")] for part in a.split.split("/"))
    cfg = {"model_split": {"online": on_split, "target": tg_split},
           "runtime": {"num_ubatch": ub, "bwd_split": split, "dp_replicas": dp, "dtype": "bf16",
                       "fused": not a.no_fused, "channels_last": True, "max_inflight": 3, "timeout_s": 300,
                       "peer_memory": not a.no_peer, "cuda_graphs": a.cuda_graphs},
           "train": {"deferred_batch_norm": True}}
    prof = None
    if a.trace:
        from tspipe_b200.profiler import TSPipeProfiler
        prof = TSPipeProfiler(filename=f"/tmp/bench_trace_{rank}.csv").__enter__()
    tsp = TSPipe(online, target, predictor, opt, byol_loss, ema_update, 0.996, "", config=cfg, device=dev,
                 profiler=prof)
    topo = tsp.topo
    replica_batch = global_batch // dp
    shape = (replica_batch, 3, a.image, a.image)
    g = torch.Generator().manual_seed(1234 + topo.replica)
    n_host = 2
    host_views = dev_views = None
    if topo.is_first:
        host_views = [(torch.randn(shape, generator=g).pin_memory(), torch.randn(shape, generator=g).pin_memory())
                      for _ in range(n_host)]
        dev_views = [(h[0].to(dev), h[1].to(dev)) for h in host_views]
    in_bytes = 2 * replica_batch * 3 * a.image * a.image * 4

    def feed(i, host):
        if topo.is_first:
            v = (host_views if host else dev_views)[i % n_host]
            return tsp.feed(v[0], v[1])
        return tsp.feed(None, None)

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
    if prof is not None:
        prof.device_events.clear()
    ms, wall_ms, losses, clocks, launches = timed(a.steps, False, ClockSampler(local) if rank == 0 else None)
    if prof is not None:
        tot = {}
        for op, row, dms in prof.device_times():
            tot[op] = tot.get(op, 0.0) + dms
        print(f"[trace rank {rank} stage {topo.stage} replica {topo.replica}] per-step device ms: " +
              ", ".join(f"{k}={v / a.steps:.2f}" for k, v in sorted(tot.items())), flush=True)
        prof.device_events.clear()
    out = {"value": round(global_batch * a.steps / (ms / 1e3), 2), "ms_per_step": round(ms / a.steps, 3),
           "gpu_launches": launches, "clocks": clocks, "parallelism": f"dp{dp}xpp{pp}", "microbatches": ub,
           "bwd_split": split, "global_batch": global_batch, "merged_views": bool(tsp.engine.merge_views), "last_loss": round(losses[-1], 5) if losses else None}
    if e2e:
        for i in range(min(a.warmup, 3)):
            feed(i, True)
        tsp.flush()
        ms2, wall2, losses2, _, _ = timed(a.steps, True)
        out["e2e"] = {"value": round(global_batch * a.steps / (max(ms2, wall2) / 1e3), 2), "unit": "images/s",
                      "h2d_bytes_per_step": in_bytes * dp, "d2h_bytes_per_step": 4 * dp,
                      "ms_per_step": round(max(ms2, wall2) / a.steps, 3),
                      "api": "TSPipe.feed(pinned host views) per step; loss read back per step; TSPipe.flush at the end"}
    tsp.stop()
    if prof is not None:
        prof.__exit__(None, None, None)
    del tsp, online, target, predictor, opt, host_views, dev_views
    gc.collect()
    torch.cuda.empty_cache()
    return out


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
    pp, dp, ub, split = default_grid(world)
    if a.pp:
        pp, dp = a.pp, world // a.pp
        ub = 1          # larger kernels beat finer interleaving on this GPU: pp2 at 2 microbatches 60.2 ms, at 1 48.1 ms
    ub = a.ubatch or ub
    split = a.bwd_split or split
    r = measure(a, pp, dp, ub, split, e2e=not a.no_e2e)
    out = {"metric": "BYOL ResNet-50 training throughput", "value": r["value"], "unit": "images/s",
           "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": r["ms_per_step"],
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "impl": "ours", "gpu_launches": r["gpu_launches"], "clocks": r["clocks"],
           "config": {"model": f"byol_{a.model}+mlp4096-256", "global_batch": r["global_batch"], "seq_len": None,
                      "image": a.image, "parallelism": r["parallelism"], "microbatches": r["microbatches"],
                      "bwd_split": r["bwd_split"], "optimizer": "LARS", "ema": 0.996,
                      "views": "both views of a network in one stacked forward, BatchNorm statistics per view"
                               if r.get("merged_views") else "one forward per view",
                      "l2_policy": "inputs larger than L2 (154 MB per replica step)",
                      "timing": "CUDA events on the compute stream around K feeds + flush, max over ranks"}}
    if r.get("last_loss") is not None:
        out["last_loss"] = r["last_loss"]
    if "e2e" in r:
        out["e2e"] = r["e2e"]
    if world >= 2 and pp == 1 and not a.no_pipeline:
        # the same job on the interleaved two-stage teacher/student pipeline (x world/2 replicas)
        p2 = measure(a, 2, world // 2, 1, split, e2e=False)
        out["pipeline"] = {k: p2[k] for k in ("value", "ms_per_step", "parallelism", "microbatches", "gpu_launches")}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
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
        from run_reference import run_reference
        return run_reference(a)
    if a.gpus > 1 and "RANK" not in os.environ:
        return relaunch(a)
    run_ours(a)


if __name__ == "__main__":
    main()
