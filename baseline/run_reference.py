"""Reference arm of ``bench.py``: the unmodified reference package, through its own public API.

``baseline/_ref`` holds the reference's sources exactly as published (``tspipe``, ``dataset`` and its
BYOL benchmark as ``tspipe_ref_byol``), installed with pip from a copy that only adds packaging
metadata.  This harness does what the reference's own ``benchmarks/byol/main.py`` +
``trainer.py:214-280`` do - build ResNet-50 + heads with the reference's model classes, its LARS, its
``TSPipeBYOLTrainer.contrastive_loss`` / ``calculate_target_network_parameters`` callbacks, construct
``tspipe.TSPipe`` and call ``feed`` with shared-memory synthetic views - minus dataset, TensorBoard and
tqdm.  Nothing from ``tspipe_b200`` is imported on this path.

Configuration: fp32 as shipped (the reference has no mixed-precision path in its pipeline), one
pipeline over all N GPUs with its fixed N-1 microbatches; for N = 1 its GPipe-emulation mode with one
microbatch, because its scheduler needs at least two stages (``tspipe/tspipe.py:106-111``).  A second run
(``reference_bf16`` in the output line) gives the reference the precision the own arm computes in: every child of
the Sequentials handed to the stock ``tspipe.TSPipe`` is wrapped so that its forward runs under
``torch.autocast(bfloat16)`` (``baseline/ref_wrappers.py``); nothing under ``baseline/_ref`` is edited.

Timing: the reference reports each batch's loss to the feeding process after a device synchronisation
(``tspipe/gpu_task.py:180,204``).  The harness records the host time at which ``feed`` hands back the
loss of each batch and reports ``t(loss of batch W+K) - t(loss of batch W)``: K steady-state steps.
Device events are not available across the reference's worker processes.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

SPLITS = {   # 30 online children (26 + 4 predictor) / 26 target children
    1: ([30], [26]),
    2: ([8, 22], [8, 18]),
    4: ([6, 5, 7, 12], [6, 5, 7, 8]),
    8: ([5, 2, 3, 3, 3, 3, 4, 7], [5, 2, 3, 3, 3, 3, 4, 3]),
}


def unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)


def run_reference(a) -> None:
    """Called by ``bench.py --impl reference`` (on every rank when launched by torchrun)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return                      # the reference spawns its own workers from one process
    if not os.path.isdir(os.path.join(REF, "tspipe")):
        return unavailable("baseline/_ref is missing: the reference is not installed on this machine")
    env = {k: v for k, v in os.environ.items()
           if not (k.startswith("TORCHELASTIC") or k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE",
                                                         "GROUP_RANK", "ROLE_RANK", "MASTER_ADDR", "MASTER_PORT",
                                                         "GROUP_WORLD_SIZE", "ROLE_WORLD_SIZE", "ROLE_NAME",
                                                         "OMP_NUM_THREADS"))}
    env["CUDA_VISIBLE_DEVICES"] = ",".join(str(i) for i in range(a.gpus))
    per_gpu = getattr(a, "per_gpu_batch", 0) or 128
    want = getattr(a, "ref_dtype", "auto")
    if want == "auto":
        # the second (bf16-autocast) run doubles the arm's time; the reference needs minutes per run on 4+ GPUs, so
        # the precision bracket is taken where it is cheap
        want = "both" if a.gpus <= 2 else "fp32"

    def one(dtype: str):
        """Run the reference once in a fresh process group; returns (json line or None, failure text)."""
        cmd = [sys.executable, os.path.abspath(__file__), "--gpus", str(a.gpus), "--steps", str(a.steps),
               "--warmup", str(a.warmup), "--per-gpu-batch", str(per_gpu), "--ref-dtype", dtype]
        limit = int(os.environ.get("TSPIPE_REF_TIMEOUT", 600))
        import signal
        proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                                start_new_session=True)
        try:
            out, err = proc.communicate(timeout=limit)
        except subprocess.TimeoutExpired:
            out, err = "", ""
        finally:
            try:                        # the reference leaves worker processes behind when it fails
                os.killpg(proc.pid, signal.SIGKILL)
            except ProcessLookupError:
                pass
        if proc.poll() is None:
            proc.wait()
        log = os.environ.get("TSPIPE_REF_LOG")
        if log:
            with open(log + ("" if dtype == "fp32" else "." + dtype), "w") as f:
                f.write(out + "\n---- stderr ----\n" + err)
        if not out and not err:
            return None, f"the reference run did not finish within {limit} s on {a.gpus} GPU(s)"
        line = next((l for l in reversed(out.splitlines()) if l.startswith('{"metric"')), None)
        if line is None:
            tail = (err or out).strip().splitlines()[-3:]
            return None, f"the reference run failed (exit {proc.returncode}): {' | '.join(tail)}"
        return line, ""

    line, why = one("bf16" if want == "bf16" else "fp32")
    if line is None:
        return unavailable(why)
    if want == "both":
        line16, why16 = one("bf16")
        rec = json.loads(line)
        if line16 is not None:
            r16 = json.loads(line16)
            rec["reference_bf16"] = {k: r16[k] for k in ("value", "unit", "ms_per_step", "dtype")}
        else:
            rec["reference_bf16"] = {"unavailable": why16[:300]}
        line = json.dumps(rec)
    print(line, flush=True)


# -------------------------------------------------------------------------------------------------
def child() -> None:
    import argparse
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, required=True)
    p.add_argument("--steps", type=int, required=True)
    p.add_argument("--warmup", type=int, required=True)
    p.add_argument("--per-gpu-batch", type=int, default=128)
    p.add_argument("--ref-dtype", default="fp32", choices=["fp32", "bf16"])
    a, _ = p.parse_known_args()

    sys.path.insert(0, HERE)
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(REF, "tspipe_ref_byol"))
    import torch
    import yaml
    n = a.gpus
    assert torch.cuda.device_count() == n, f"{torch.cuda.device_count()} GPUs visible, expected {n}"
    on_split, tg_split = SPLITS[n]
    cfg = {"tspipe": {
        "train": {"deferred_batch_norm": True, "save_model_every_iter": 0},
        "model_split": {"online": on_split, "target": tg_split},
        "optimizer": {"skip_optimizer": False, "num_skip_initial_staleness": 0, "gradient_accumulation": 1,
                      "reduce_verbose": False},
        "gpipe_emulation": {"enabled": n == 1, "num_ubatch": 1},
        "async_param_update_emulation": {"enabled": False}}}
    work = tempfile.mkdtemp(prefix="tspipe_ref_")
    cfg_path = os.path.join(work, "tspipe.yaml")
    with open(cfg_path, "w") as f:
        yaml.safe_dump(cfg, f)
    os.chdir(work)
    sys.argv = [sys.argv[0], f"--tspipe-config={cfg_path}", "--ip=127.0.0.1", "--rank=0", "--num-nodes=1"]

    # the reference's own model / optimizer / callbacks
    from models.mlp_head import MLPHead
    from models.resnet_base_network import ResNet18
    from main import LARS
    from trainer import TSPipeBYOLTrainer
    import tspipe

    torch.manual_seed(0)
    head = {"mlp_hidden_size": 4096, "projection_size": 256}
    online = ResNet18(name="resnet50", projection_head=head)
    predictor = MLPHead(in_channels=256, **head)
    target = ResNet18(name="resnet50", projection_head=head)
    for q, k in zip(online.parameters(), target.parameters()):
        k.data.copy_(q.data)
        k.requires_grad = False
    online, target, predictor = online.to_sequential(), target.to_sequential(), predictor.to_sequential()
    # The reference chains the children of the online net and the predictor into one name -> module dict
    # (`tspipe/tspipe.py:553-580`); the predictor's default names "0".."3" would overwrite the first online
    # layers whenever both end up in one partition (always the case on 1 GPU), so give them names of their own.
    from collections import OrderedDict
    predictor = torch.nn.Sequential(OrderedDict((f"pred{i}", m) for i, m in enumerate(predictor.children())))
    if a.ref_dtype == "bf16":
        from ref_wrappers import autocast_children
        online, target, predictor = autocast_children(online), autocast_children(target), autocast_children(predictor)
    batch = a.per_gpu_batch * n
    opt = LARS(list(online.parameters()) + list(predictor.parameters()), lr=0.2 * batch / 256, momentum=0.9,
               weight_decay=1.5e-6)
    tsp = tspipe.TSPipe(online, target, predictor, opt, TSPipeBYOLTrainer.contrastive_loss,
                        TSPipeBYOLTrainer.calculate_target_network_parameters, 0.996, work)
    if not tsp.is_primary:
        return
    g = torch.Generator().manual_seed(1234)
    v1 = torch.randn(batch, 3, 224, 224, generator=g).share_memory_()
    v2 = torch.randn(batch, 3, 224, 224, generator=g).share_memory_()
    W, K = a.warmup, a.steps
    stamp = {}
    total = W + K + 10                     # the loss of batch b comes back several feeds later
    for i in range(total):
        tsp.feed(v1, v2)
        b = tsp.forward_complete_batch_idx
        if b and b not in stamp:
            stamp[b] = time.perf_counter()
        if W + K in stamp:
            break
    deadline = time.time() + 600
    while W + K not in stamp and time.time() < deadline:
        l = tsp.wait_forward()
        b = tsp.forward_complete_batch_idx
        if b and b not in stamp:
            stamp[b] = time.perf_counter()
        if l is None:
            time.sleep(0.001)
    ok = W in stamp and (W + K) in stamp
    if ok:
        dt = stamp[W + K] - stamp[W]
        out = {"metric": "BYOL ResNet-50 training throughput", "value": round(batch * K / dt, 2), "unit": "images/s",
               "n_gpus": n, "steps": K, "warmup": W, "ms_per_step": round(dt / K * 1e3, 3), "higher_is_better": True,
               "scaling": "weak", "vs_baseline": None,
               "dtype": "fp32 (as shipped; TF32 convolutions by PyTorch default)" if a.ref_dtype == "fp32"
                        else "bf16 (every Sequential child's forward under torch.autocast; fp32 parameters)",
               "data": "synthetic", "impl": "reference",
               "config": {"model": "byol_resnet50+mlp4096-256", "global_batch": batch, "seq_len": None, "image": 224,
                          "parallelism": f"pp{n}" + (" (gpipe_emulation)" if n == 1 else ""),
                          "microbatches": 1 if n == 1 else n - 1, "bwd_split": 1 if n == 1 else 2,
                          "optimizer": "LARS", "ema": 0.996, "views": "one forward per view",
                          "l2_policy": "inputs larger than L2 (a step's activations are several GB per GPU)",
                          "timing": "host time between the arrivals of the losses of batch W and batch W+K"},
               # the reference's number IS end to end: every step its feed() ships the two fp32 views from shared
               # host memory to the first stage and the loss comes back to the feeding process as a Python float
               "e2e": {"value": round(batch * K / dt, 2), "unit": "images/s", "ms_per_step": round(dt / K * 1e3, 3),
                       "h2d_bytes_per_step": 2 * batch * 3 * 224 * 224 * 4, "d2h_bytes_per_step": 4,
                       "api": "tspipe.TSPipe.feed(shared-memory host views) per step; loss float back per step"}}
        print(json.dumps(out), flush=True)
    try:
        tsp.stop()
    except BaseException as e:  # noqa: BLE001
        print(f"reference stop() raised {e!r}", file=sys.stderr)
    if not ok:
        sys.exit(3)
    os._exit(0)


if __name__ == "__main__":
    child()
