"""Two-GPU pipeline checks (NCCL links, peer-mapped buffers) against the single-process oracle."""
import copy
from argparse import Namespace

import pytest
import torch
from torch import nn

from tests.helpers import run_ranks

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _ssl_models():
    from tspipe_b200.models.mlp import mlp_sequential
    torch.manual_seed(0)
    online = mlp_sequential([48, 64, 64, 48, 32], batch_norm=True)
    target = copy.deepcopy(online)
    predictor = nn.Sequential(nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 32))
    return online, target, predictor


def _batches(n):
    g = torch.Generator().manual_seed(1)
    return [(torch.randn(32, 48, generator=g), torch.randn(32, 48, generator=g)) for _ in range(n)]


def _byol_rank(rank, world, n_steps):
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.optim import LARS
    from tspipe_b200.runtime.engine import CrossStageEmaTeacher
    online, target, predictor = _ssl_models()
    opt = LARS(list(online.parameters()) + list(predictor.parameters()), lr=0.2, weight_decay=1e-4, momentum=0.9)
    cfg = {"model_split": {"online": [4, 4], "target": [3, 2]},     # different cuts: the EMA crosses GPUs
           "runtime": {"num_ubatch": 2, "bwd_split": 2, "dtype": "fp32", "timeout_s": 120},
           "train": {"deferred_batch_norm": False}}
    tsp = TSPipe(online, target, predictor, opt, byol_loss, ema_update, 0.9, "", config=cfg, device=f"cuda:{rank}")
    upd = tsp.engine.updater
    info = (type(upd).__name__, getattr(upd, "peer_flats", None) is not None)
    losses = []
    for a, b in _batches(n_steps):
        l = tsp.feed(a.pin_memory(), b.pin_memory()) if rank == 0 else tsp.feed(None, None)
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    on, tg = tsp.state_dicts()
    dist.destroy_process_group()
    return losses, on, tg, info


def test_byol_two_stage_pipeline_with_cross_gpu_momentum_update():
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.optim import LARS
    from tspipe_b200.oracle import DelayedTeacherOracle
    n_steps = 5
    online, target, predictor = _ssl_models()
    full = nn.Sequential(*list(online.children()), *list(predictor.children()))
    opt = LARS(list(full.parameters()), lr=0.2, weight_decay=1e-4, momentum=0.9)
    orc = DelayedTeacherOracle(full, target, opt, byol_loss, ema_update, 0.9, kd=False, n_ubatch=2, bwd_split=2)
    n_t = len(list(target.parameters()))
    f = orc.update_fn
    orc.update_fn = lambda m, on, tg: f(m, on[:n_t], tg)
    ref = [orc.step(a, b) for a, b in _batches(n_steps)]
    out = run_ranks(_byol_rank, 2, n_steps)
    assert out[1][3] == ("CrossStageEmaTeacher", True) or out[0][3] == ("CrossStageEmaTeacher", True)
    torch.testing.assert_close(torch.tensor(out[1][0]), torch.tensor(ref), rtol=2e-4, atol=1e-5)
    torch.testing.assert_close(torch.tensor(out[0][0]), torch.tensor(ref), rtol=2e-4, atol=1e-5)   # forwarded to rank 0
    got_t = [v for j in sorted(out[0][2]) for k, v in out[0][2][j].items() if "running" not in k and "num_batches" not in k]
    for a, b in zip(got_t, list(orc.final_teacher().values())):
        torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-5)


def _moco_models(dim=64):
    from tspipe_b200.models.mlp import mlp_sequential
    torch.manual_seed(3)
    online = mlp_sequential([32, 64, dim])
    target = copy.deepcopy(online)
    predictor = nn.Sequential(nn.Linear(dim, 64), nn.Tanh(), nn.Linear(64, dim))
    return online, target, predictor


def _moco_batches(n):
    g = torch.Generator().manual_seed(4)
    return [(torch.randn(256, 32, generator=g), torch.randn(256, 32, generator=g)) for _ in range(n)]


def _moco_rank(rank, world, n_steps, dim=64):
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import ema_update, moco_loss
    online, target, predictor = _moco_models(dim)
    opt = torch.optim.SGD(list(online.parameters()) + list(predictor.parameters()), lr=0.2)
    cfg = {"model_split": {"online": [6], "target": [3]},
           "runtime": {"num_ubatch": 2, "bwd_split": 1, "dtype": "fp32", "dp_replicas": 2, "timeout_s": 120},
           "train": {"deferred_batch_norm": False}}
    tsp = TSPipe(online, target, predictor, opt, moco_loss, ema_update, 0.9, "", config=cfg, device=f"cuda:{rank}",
                 extra_args=Namespace(moco_t=0.2))
    losses = []
    for a, b in _moco_batches(n_steps):
        sl = slice(rank * 128, (rank + 1) * 128)
        l = tsp.feed(a[sl].pin_memory(), b[sl].pin_memory())
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    from tspipe_b200.ops import gemm
    gemm.check_status()
    dist.destroy_process_group()
    return losses


@pytest.mark.parametrize("dim", [64, 256])
def test_moco_replicas_gather_keys_through_peer_memory_and_tcgen05_logits(dim):
    """dim 64: gathered-key tcgen05 GEMM + CE kernel; dim 256: the fused attention-style kernel that streams key
    tiles from both replicas' buffers and never writes the logits."""
    from tspipe_b200.losses import ema_update, moco_loss
    from tspipe_b200.oracle import DelayedTeacherOracle
    n_steps = 3
    online, target, predictor = _moco_models(dim)
    full = nn.Sequential(*list(online.children()), *list(predictor.children()))
    opt = torch.optim.SGD(full.parameters(), lr=0.2)
    orc = DelayedTeacherOracle(full, target, opt, moco_loss, ema_update, 0.9, kd=False, n_ubatch=4, bwd_split=1,
                               extra_args=Namespace(moco_t=0.2))
    n_t = len(list(target.parameters()))
    f = orc.update_fn
    orc.update_fn = lambda m, on, tg: f(m, on[:n_t], tg)
    ref = [orc.step(a, b) for a, b in _moco_batches(n_steps)]
    out = run_ranks(_moco_rank, 2, n_steps, dim)
    mean = [(x + y) / 2 for x, y in zip(out[0], out[1])]
    torch.testing.assert_close(torch.tensor(mean), torch.tensor(ref), rtol=2e-2, atol=2e-2)   # bf16 logits


def _kd_batches(n):
    g = torch.Generator().manual_seed(7)
    return [(torch.randn(64, 3, 32, 32, generator=g), torch.randint(0, 10, (64,), generator=g)) for _ in range(n)]


def _split_rank(rank, world, n_steps):
    import warnings
    import torch.distributed as dist
    from tspipe_b200 import TSPipe, TSPipeMode
    from tspipe_b200.losses import soft_target_kd
    from tspipe_b200.models.mlp import toy_student, toy_teacher
    torch.manual_seed(0)
    teacher, student = toy_teacher(), toy_student()
    opt = torch.optim.SGD(student.parameters(), lr=0.05)
    cfg = {"model_split": {"online": [5], "target": [9]},
           "runtime": {"num_ubatch": 4, "dtype": "fp32", "timeout_s": 120, "placement": "split"},
           "train": {"deferred_batch_norm": False}}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(student, teacher, None, opt, soft_target_kd, None, 1.0, "", config=cfg, device=f"cuda:{rank}",
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False,
                     extra_args=Namespace(T=4.0, alpha=0.9))
    losses = []
    for x, y in _kd_batches(n_steps):
        l = tsp.feed(x.pin_memory(), x.pin_memory(), y.pin_memory())
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    peer = getattr(tsp.engine, "peer", False)
    dist.destroy_process_group()
    return losses, peer


def test_split_placement_kd_loss_reads_teacher_logits_from_peer_gpu():
    """Teacher on cuda:0, student on cuda:1: the fused KD loss kernel on cuda:1 reads the teacher logits from
    the ring buffer in cuda:0's memory."""
    from tspipe_b200.losses import soft_target_kd
    from tspipe_b200.models.mlp import toy_student, toy_teacher
    from tspipe_b200.oracle import DelayedTeacherOracle
    n_steps = 5
    torch.manual_seed(0)
    teacher, student = toy_teacher(), toy_student()
    opt = torch.optim.SGD(student.parameters(), lr=0.05)
    orc = DelayedTeacherOracle(student, teacher, opt, soft_target_kd, None, 1.0, kd=True, n_ubatch=4, bwd_split=1,
                               extra_args=Namespace(T=4.0, alpha=0.9))
    ref = [orc.step(x, x, y) for x, y in _kd_batches(n_steps)]
    out = run_ranks(_split_rank, 2, n_steps)
    assert out[1][1] is True
    torch.testing.assert_close(torch.tensor(out[1][0]), torch.tensor(ref), rtol=2e-4, atol=1e-5)
