"""The training entry points under ``benchmarks/`` run end to end (tiny models, CPU, gloo)."""
import os
import subprocess
import sys

import pytest

from tests.helpers import free_port

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write(tmp_path, name, text):
    p = tmp_path / name
    p.write_text(text)
    return str(p)


def _run(cmd, nproc=1, timeout=240):
    env = dict(os.environ, TSPIPE_NO_AFFINITY="1", OMP_NUM_THREADS="1")
    full = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
            "--master-addr", "127.0.0.1", "--master-port", str(free_port())] + cmd
    res = subprocess.run(full, env=env, capture_output=True, text=True, timeout=timeout, cwd=REPO)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    return res.stdout


def _check_run_artifacts(path, min_losses):
    """The applications leave TensorBoard-style scalars (always as ``scalars.csv``) and a final ``model.pth`` with the
    reference's three keys, whose network state dicts cover the whole networks (all partitions joined)."""
    import torch
    rows = [l.split(",") for l in (path / "scalars.csv").read_text().splitlines()[1:]]
    losses = [float(r[3]) for r in rows if r[2] == "loss"]
    assert len(losses) >= min_losses and all(v == v for v in losses)
    sd = torch.load(path / "model.pth", weights_only=False)
    assert set(sd) == {"online_network_state_dict", "target_network_state_dict", "optimizer_state_dict"}
    assert len(sd["online_network_state_dict"]) > 0 and len(sd["target_network_state_dict"]) > 0
    assert any(f.name.startswith("events.out.tfevents") for f in path.iterdir())


def test_distilbert_app_two_stage_pipeline(tmp_path):
    cfg = _write(tmp_path, "t.yaml", """
tspipe:
  train: {deferred_batch_norm: False}
  model_split: {online: [2, 1], target: [2, 2]}
  runtime: {num_ubatch: 2, bwd_split: 2, backend: gloo, timeout_s: 60}
""")
    out = _run(["benchmarks/distilbert/train.py", "--teacher", "tiny", "--batch-size", "8", "--seq-len", "16",
                "--iters", "12", "--tspipe-config", cfg, "--artifact-dir", str(tmp_path)], nproc=2)
    assert "iter 10 loss" in out
    _check_run_artifacts(tmp_path, min_losses=8)


def test_soft_target_app_single_stage(tmp_path):
    cfg = _write(tmp_path, "t.yaml", """
tspipe:
  train: {deferred_batch_norm: False}
  model_split: {online: [8], target: [8]}
  runtime: {num_ubatch: 2, bwd_split: 1, backend: gloo, timeout_s: 60}
""")
    out = _run(["benchmarks/soft_target/train_kd.py", "--t-name", "vit_tiny_test", "--s-name", "vit_tiny_test",
                "--image", "32", "--num-class", "10", "--batch-size", "8", "--iters-per-epoch", "11",
                "--tspipe-config", cfg, "--artifact-dir", str(tmp_path)])
    assert "iter 10 loss" in out
    _check_run_artifacts(tmp_path, min_losses=8)


def test_moco_app_with_replicas(tmp_path):
    cfg = _write(tmp_path, "t.yaml", """
tspipe:
  train: {deferred_batch_norm: True}
  model_split: {online: [20], target: [15]}
  runtime: {num_ubatch: 2, bwd_split: 1, backend: gloo, dp_replicas: 2, timeout_s: 60}
""")
    out = _run(["benchmarks/moco_v3/main.py", "--arch", "vit_tiny_test", "--image", "32", "--batch-size", "8",
                "--moco-dim", "32", "--moco-mlp-dim", "64", "--max-iters", "11", "--dummy",
                "--tspipe-config", cfg, "--artifact-dir", str(tmp_path)], nproc=2)
    assert "iter 10 loss" in out
    _check_run_artifacts(tmp_path, min_losses=8)


def test_byol_app_two_stages(tmp_path):
    cfg = _write(tmp_path, "t.yaml", """
tspipe:
  train: {deferred_batch_norm: True, save_model_every_iter: 5}
  model_split: {online: [6, 16], target: [6, 12]}
  runtime: {num_ubatch: 2, bwd_split: 2, backend: gloo, timeout_s: 60}
""")
    app = _write(tmp_path, "c.yaml", """
network: {name: resnet18, projection_head: {mlp_hidden_size: 32, projection_size: 16}}
data_transforms: {input_shape: "(32,32,3)"}
dataset: {name: dummy, path: ""}
trainer: {batch_size: 8, m: 0.99, max_epochs: 1, num_workers: 0, dummy_input: True, optimizer_type: lars}
optimizer: {params: {lr: 0.1, momentum: 0.9, weight_decay: 0.000001}}
""")
    out = _run(["benchmarks/byol/main.py", "--config", app, "--tspipe-config", cfg, "--max-iters", "12",
                "--artifact-dir", str(tmp_path)], nproc=2)
    assert "iter 10 loss" in out
    assert (tmp_path / "model_batch5_part0.pt").exists() and (tmp_path / "model_batch10_part1.pt").exists()
    assert (tmp_path / "profile_out.csv").exists()
    _check_run_artifacts(tmp_path, min_losses=8)


def test_plain_trainer_equals_the_oracle_with_an_immediate_teacher():
    """The non-pipelined trainer (``--plain`` in the applications) is the oracle without delay: one microbatch, the
    teacher updated right after every optimizer step."""
    import copy
    import torch
    from torch import nn
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.models.mlp import mlp_sequential
    from tspipe_b200.oracle import DelayedTeacherOracle
    from tspipe_b200.plain_trainer import PlainTrainer

    def models():
        torch.manual_seed(0)
        online = mlp_sequential([24, 32, 16], batch_norm=True)
        return online, copy.deepcopy(online), nn.Sequential(nn.Linear(16, 16), nn.ReLU(), nn.Linear(16, 16))
    g = torch.Generator().manual_seed(1)
    batches = [(torch.randn(12, 24, generator=g), torch.randn(12, 24, generator=g)) for _ in range(5)]

    online, target, pred = models()
    full = nn.Sequential(*list(online.children()), *list(pred.children()))
    opt = torch.optim.SGD(full.parameters(), lr=0.1, momentum=0.9)
    orc = DelayedTeacherOracle(full, target, opt, byol_loss, ema_update, 0.9, kd=False, n_ubatch=1, bwd_split=1, gpipe=True)
    n_t = len(list(target.parameters()))
    fn = orc.update_fn
    orc.update_fn = lambda m, on, tg: fn(m, on[:n_t], tg)
    want = [orc.step(a, b) for a, b in batches]

    online, target, pred = models()
    opt = torch.optim.SGD(list(online.parameters()) + list(pred.parameters()), lr=0.1, momentum=0.9)
    tr = PlainTrainer(online, target, pred, opt, byol_loss, ema_update, 0.9, device="cpu")
    got = [tr.feed(a, b) for a, b in batches]
    assert tr.stop() == [] and tr.meter.samples == 60
    torch.testing.assert_close(torch.tensor(got), torch.tensor(want), rtol=1e-5, atol=1e-6)
    on, tg = tr.state_dicts()
    for a, b in zip([v for k, v in tg[0].items() if "running" not in k and "num_batches" not in k],
                    orc.final_teacher().values()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_byol_app_plain_trainer(tmp_path):
    app = _write(tmp_path, "c.yaml", """
network: {name: resnet18, projection_head: {mlp_hidden_size: 32, projection_size: 16}}
data_transforms: {input_shape: "(32,32,3)"}
dataset: {name: dummy, path: ""}
trainer: {batch_size: 8, m: 0.99, max_epochs: 1, num_workers: 0, dummy_input: True, optimizer_type: lars}
optimizer: {params: {lr: 0.1, momentum: 0.9, weight_decay: 0.000001}}
""")
    env = dict(os.environ, TSPIPE_NO_AFFINITY="1", OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    res = subprocess.run([sys.executable, "benchmarks/byol/main.py", "--config", app, "--plain", "--max-iters", "11",
                          "--artifact-dir", str(tmp_path)], env=env, capture_output=True, text=True, timeout=240, cwd=REPO)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "iter 10 loss" in res.stdout
    _check_run_artifacts(tmp_path, min_losses=10)
