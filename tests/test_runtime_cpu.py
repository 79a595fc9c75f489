"""Pipelined runtime on CPU/gloo against the single-process delayed-teacher oracle."""
import copy
from argparse import Namespace

import pytest
import torch
from torch import nn

from tests.helpers import run_ranks
from tspipe_b200 import TSPipe, TSPipeMode
from tspipe_b200.losses import byol_loss, ema_update, soft_target_kd
from tspipe_b200.models.mlp import mlp_sequential, toy_student, toy_teacher
from tspipe_b200.oracle import DelayedTeacherOracle

KD_ARGS = Namespace(T=4.0, alpha=0.9)


def _toy_batches(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(64, 3, 32, 32, generator=g), torch.randint(0, 10, (64,), generator=g)) for _ in range(n)]


def _oracle_kd(n_steps, n_ubatch, bwd_split, **kw):
    torch.manual_seed(0)
    teacher, student = toy_teacher(), toy_student()
    opt = torch.optim.SGD(student.parameters(), lr=0.05)
    orc = DelayedTeacherOracle(student, teacher, opt, soft_target_kd, None, 1.0, kd=True, n_ubatch=n_ubatch,
                               bwd_split=bwd_split, extra_args=KD_ARGS, **kw)
    losses = [orc.step(x, x, y) for x, y in _toy_batches(n_steps)]
    return losses, {k: v.detach().clone() for k, v in student.state_dict().items()}


def test_toy_kd_two_process_pipeline_matches_oracle(tmp_path):
    """Toy soft-target KD, two pipeline stages as two spawned CPU processes (gloo), batch 64 in four
    microbatches, SGD lr 0.05, seed 0: losses and final student weights equal the oracle's."""
    n_steps = 6
    ref_losses, ref_state = _oracle_kd(n_steps, 4, 2)
    torch.manual_seed(0)
    teacher, student = toy_teacher(), toy_student()
    opt = torch.optim.SGD(student.parameters(), lr=0.05)
    cfg = {"model_split": {"online": [3, 2], "target": [5, 4]}, "runtime": {"num_ubatch": 4, "backend": "gloo", "timeout_s": 60},
           "train": {"deferred_batch_norm": False}}
    with pytest.warns(UserWarning):
        tsp = TSPipe(student, teacher, None, opt, soft_target_kd, None, 1.0, str(tmp_path),
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False, extra_args=KD_ARGS,
                     config=cfg, argv=["--ip", "127.0.0.1", "--rank", "0", "--num-nodes", "1"], device="cpu")
    losses = []
    for x, y in _toy_batches(n_steps):
        l = tsp.feed(x, x, y)
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    assert len(losses) == n_steps
    torch.testing.assert_close(torch.tensor(losses), torch.tensor(ref_losses), rtol=1e-5, atol=1e-6)
    online, _ = tsp.state_dicts()
    merged = {}
    for st in online.values():
        merged.update(st)
    assert set(merged) == set(ref_state)
    for k in ref_state:
        torch.testing.assert_close(merged[k], ref_state[k], rtol=1e-5, atol=1e-6)


# ---------------------------------------------------------------------------------------------
def _ssl_models(seed=0):
    torch.manual_seed(seed)
    online = mlp_sequential([48, 32, 32, 24, 16], batch_norm=True)
    target = copy.deepcopy(online)
    predictor = nn.Sequential(nn.Linear(16, 16), nn.ReLU(), nn.Linear(16, 16))
    return online, target, predictor


def _ssl_batches(n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(24, 48, generator=g), torch.randn(24, 48, generator=g)) for _ in range(n)]


def _ssl_rank(rank, world, cfg, n_steps):
    online, target, predictor = _ssl_models()
    opt = torch.optim.SGD(list(online.parameters()) + list(predictor.parameters()), lr=0.1, momentum=0.9)
    tsp = TSPipe(online, target, predictor, opt, byol_loss, ema_update, 0.9, "", config=cfg, device="cpu")
    losses = []
    for i, (a, b) in enumerate(_ssl_batches(n_steps)):
        if i == 3:
            tsp.update_lr(0.05)
            tsp.update_momentum(0.95)
        l = tsp.feed(a, b)
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    on, tg = tsp.state_dicts()
    return losses, on, tg


def _ssl_oracle(n_steps, n_ubatch, bwd_split, skip=0, gpipe=False):
    from tspipe_b200.batchnorm import DeferredBatchNorm
    online, target, predictor = _ssl_models()
    full = nn.Sequential(*list(online.children()), *list(predictor.children()))
    opt = torch.optim.SGD(list(online.parameters()) + list(predictor.parameters()), lr=0.1, momentum=0.9)
    orc = DelayedTeacherOracle(full, target, opt, byol_loss, ema_update, 0.9, kd=False, n_ubatch=n_ubatch,
                               bwd_split=bwd_split, skip_staleness=skip, gpipe=gpipe)
    n_t = len(list(target.parameters()))
    orc_update = orc.update_fn
    orc.update_fn = lambda m, on, tg: orc_update(m, on[:n_t], tg)
    losses = []
    for i, (a, b) in enumerate(_ssl_batches(n_steps)):
        if i == 3:
            for g in opt.param_groups:
                g["lr"] = 0.05
            orc.momentum = 0.95
        losses.append(orc.step(a, b))
    return losses, orc.final_teacher(), {k: v.detach() for k, v in full.state_dict().items()}


@pytest.mark.parametrize("pp,n_ub,split,skip,gpipe", [(2, 2, 2, 0, False), (3, 2, 2, 0, False), (3, 3, 1, 1, False),
                                                      (2, 2, 1, 0, True), (1, 2, 2, 0, False)])
def test_ssl_momentum_pipeline_matches_oracle(pp, n_ub, split, skip, gpipe):
    """BYOL-style run (BatchNorm, predictor, SGD momentum, EMA teacher, lr/momentum updates) in
    launcher mode: the pipelined result equals the oracle with the one-step-delayed teacher."""
    n_steps = 7
    n_on, n_tg = 5 + 3, 5
    from tspipe_b200.tspipe import default_balance
    cfg = {"model_split": {"online": default_balance(n_on, pp), "target": default_balance(n_tg, pp)},
           "runtime": {"num_ubatch": n_ub, "bwd_split": split, "backend": "gloo", "timeout_s": 60},
           "optimizer": {"num_skip_initial_staleness": skip},
           "gpipe_emulation": {"enabled": gpipe, "num_ubatch": n_ub},
           "train": {"deferred_batch_norm": False}}
    ref_losses, ref_teacher, ref_online = _ssl_oracle(n_steps, n_ub, split, skip, gpipe)
    out = run_ranks(_ssl_rank, pp, cfg, n_steps)
    losses = out[pp - 1][0]
    assert len(losses) == n_steps
    torch.testing.assert_close(torch.tensor(losses), torch.tensor(ref_losses), rtol=2e-5, atol=1e-6)
    _, on, tg = out[0]
    # teacher parameters: compare values in order (keys differ: the oracle has the full model)
    got_t = [v for j in sorted(tg) for k, v in tg[j].items() if "running" not in k and "num_batches" not in k]
    want_t = list(ref_teacher.values())
    assert len(got_t) == len(want_t)
    for a, b in zip(got_t, want_t):
        torch.testing.assert_close(a, b, rtol=2e-5, atol=1e-6)
    got_o = [v for j in sorted(on) for k, v in on[j].items() if "running" not in k and "num_batches" not in k]
    want_o = [v for k, v in ref_online.items() if "running" not in k and "num_batches" not in k]
    assert len(got_o) == len(want_o)
    for a, b in zip(got_o, want_o):
        torch.testing.assert_close(a, b, rtol=2e-5, atol=1e-6)


def _merge_rank(rank, world, merge, n_steps):
    cfg = {"model_split": {"online": [8], "target": [5]},
           "runtime": {"num_ubatch": 1, "bwd_split": 1, "backend": "gloo", "timeout_s": 60, "merge_views": merge},
           "train": {"deferred_batch_norm": True}}
    out = _ssl_rank(rank, world, cfg, n_steps)
    return out


def test_stacked_views_on_a_single_stage_equal_one_forward_per_view():
    """Single stage, one microbatch: both views of a network run as ONE stacked forward/backward with per-view
    BatchNorm statistics.  Losses, parameters and running statistics equal those of one forward per view and the
    losses equal the oracle's."""
    n_steps = 6
    merged = run_ranks(_merge_rank, 1, True, n_steps)[0]
    plain = run_ranks(_merge_rank, 1, False, n_steps)[0]
    ref_losses, _, _ = _ssl_oracle(n_steps, 1, 1)
    torch.testing.assert_close(torch.tensor(merged[0]), torch.tensor(ref_losses), rtol=2e-5, atol=1e-6)
    torch.testing.assert_close(torch.tensor(merged[0]), torch.tensor(plain[0]), rtol=1e-5, atol=1e-6)
    for got, want in ((merged[1], plain[1]), (merged[2], plain[2])):
        for j in want:
            assert list(got[j]) == list(want[j])
            for k in want[j]:
                torch.testing.assert_close(got[j][k], want[j][k], rtol=1e-5, atol=1e-6, msg=k)


# ---------------------------------------------------------------------------------------------
def _moco_models():
    torch.manual_seed(3)
    online = mlp_sequential([20, 32, 24, 16])
    target = copy.deepcopy(online)
    predictor = nn.Sequential(nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 16))
    return online, target, predictor


def _moco_batches(n):
    g = torch.Generator().manual_seed(4)
    return [(torch.randn(16, 20, generator=g), torch.randn(16, 20, generator=g)) for _ in range(n)]


def _moco_rank(rank, world, cfg, n_steps):
    from tspipe_b200.losses import moco_loss
    online, target, predictor = _moco_models()
    opt = torch.optim.SGD(list(online.parameters()) + list(predictor.parameters()), lr=0.2)
    tsp = TSPipe(online, target, predictor, opt, moco_loss, ema_update, 0.9, "", config=cfg, device="cpu",
                 extra_args=Namespace(moco_t=0.2))
    dp = cfg["runtime"]["dp_replicas"]
    rep = tsp.topo.replica
    losses = []
    for a, b in _moco_batches(n_steps):
        per = a.shape[0] // dp
        sl = slice(rep * per, (rep + 1) * per)
        l = tsp.feed(a[sl], b[sl]) if tsp.topo.is_first else tsp.feed(None, None)
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    return losses, tsp.state_dicts()[0], (tsp.topo.replica, tsp.topo.stage)


@pytest.mark.parametrize("pp,dp", [(1, 2), (2, 2)])
def test_moco_data_parallel_replicas_gather_keys(pp, dp):
    """MoCo-style InfoNCE with ``dp`` pipeline replicas: keys are all-gathered across replicas, gradients are
    averaged, and the result equals single-process training on the full batch."""
    from tspipe_b200.losses import moco_loss
    from tspipe_b200.tspipe import default_balance
    n_steps = 4
    online, target, predictor = _moco_models()
    full = nn.Sequential(*list(online.children()), *list(predictor.children()))
    opt = torch.optim.SGD(full.parameters(), lr=0.2)
    orc = DelayedTeacherOracle(full, target, opt, moco_loss, ema_update, 0.9, kd=False, n_ubatch=2 * dp, bwd_split=1,
                               extra_args=Namespace(moco_t=0.2))
    n_t = len(list(target.parameters()))
    f = orc.update_fn
    orc.update_fn = lambda m, on, tg: f(m, on[:n_t], tg)
    ref = [orc.step(a, b) for a, b in _moco_batches(n_steps)]
    cfg = {"model_split": {"online": default_balance(4 + 3, pp), "target": default_balance(4, pp)},
           "runtime": {"num_ubatch": 2, "bwd_split": 1, "backend": "gloo", "dp_replicas": dp, "timeout_s": 60},
           "train": {"deferred_batch_norm": False}}
    out = run_ranks(_moco_rank, pp * dp, cfg, n_steps)
    last = [o for o in out if o[2][1] == pp - 1]
    mean = [sum(x) / dp for x in zip(*[o[0] for o in last])]
    torch.testing.assert_close(torch.tensor(mean), torch.tensor(ref), rtol=2e-5, atol=1e-6)
    got = [v for j in sorted(out[0][1]) for v in out[0][1][j].values()]
    want = list(full.state_dict().values())
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b.detach(), rtol=2e-5, atol=1e-6)


# ---------------------------------------------------------------------------------------------
def _split_rank(rank, world, n_steps):
    torch.manual_seed(0)
    teacher, student = toy_teacher(), toy_student()
    opt = torch.optim.SGD(student.parameters(), lr=0.05)
    cfg = {"model_split": {"online": [3, 2], "target": [5, 4]},
           "runtime": {"num_ubatch": 4, "backend": "gloo", "timeout_s": 60, "placement": "split"},
           "train": {"deferred_batch_norm": False}}
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(student, teacher, None, opt, soft_target_kd, None, 1.0, "", config=cfg, device="cpu",
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False, extra_args=KD_ARGS)
    losses = []
    for x, y in _toy_batches(n_steps):
        l = tsp.feed(x, x, y)
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    return losses, tsp.state_dicts()[0]


def test_split_placement_teacher_and_student_on_different_ranks():
    """Toy KD with the 2-stage teacher on ranks 0-1 and the 2-stage student on ranks 2-3: same losses and
    final student weights as the oracle; rank 0 still receives the losses."""
    n_steps = 5
    ref_losses, ref_state = _oracle_kd(n_steps, 4, 1)
    out = run_ranks(_split_rank, 4, n_steps)
    torch.testing.assert_close(torch.tensor(out[3][0]), torch.tensor(ref_losses), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(torch.tensor(out[0][0]), torch.tensor(ref_losses), rtol=1e-5, atol=1e-6)
    merged = {}
    for st in out[0][1].values():
        merged.update(st)
    assert set(merged) == set(ref_state)
    for k in ref_state:
        torch.testing.assert_close(merged[k], ref_state[k], rtol=1e-5, atol=1e-6)


def _async_rank(rank, world, enabled):
    import warnings
    torch.manual_seed(0)
    student = mlp_sequential([12, 16, 4])
    teacher = mlp_sequential([12, 8, 4])
    opt = torch.optim.SGD(student.parameters(), lr=0.5)
    cfg = {"model_split": {"online": [3], "target": [3]}, "async_param_update_emulation": {"enabled": enabled},
           "runtime": {"num_ubatch": 2, "bwd_split": 1, "backend": "gloo", "timeout_s": 60},
           "train": {"deferred_batch_norm": False}}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(student, teacher, None, opt, soft_target_kd, None, 1.0, "", config=cfg, device="cpu",
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False, extra_args=KD_ARGS)
    g = torch.Generator().manual_seed(9)
    x, y = torch.randn(8, 12, generator=g), torch.randint(0, 4, (8,), generator=g)
    losses = [tsp.feed(x, x, y) for _ in range(5)]
    losses = [l for l in losses if l is not None] + tsp.stop()
    return losses


def test_async_param_update_emulation_makes_the_student_one_step_stale():
    """With the emulation on, batch b runs on the parameters of version b-2: feeding the same batch
    repeatedly, batches 1 and 2 (both on version 0) give the same loss, batch 3 (version 1) a lower one;
    without it every step improves."""
    on = run_ranks(_async_rank, 1, True)[0]
    off = run_ranks(_async_rank, 1, False)[0]
    assert len(on) == 5 and len(off) == 5
    assert abs(on[0] - on[1]) < 1e-7 and on[2] < on[1]
    assert off[1] < off[0] - 1e-4
    assert abs(on[2] - off[1]) < 1e-6          # version 1 is the same in both runs


@pytest.mark.parametrize("split_on,split_tg", [([5, 3], [3, 2]), ([8], [5]), ([3, 5], [1, 4])])
def test_split_placement_with_momentum_teacher_matches_oracle(split_on, split_tg):
    """BYOL-style run with the teacher stages on the first ranks and the student stages on the others: the student
    ranks ship the parameter runs each teacher stage needs after every optimizer step, the teacher folds step k in
    before its forward of batch k + 2.  Losses, final teacher and final student equal the oracle with the
    one-step-delayed teacher, for equal and unequal cuts (lr and momentum change on the way)."""
    n_steps, n_ub = 7, 2
    cfg = {"model_split": {"online": split_on, "target": split_tg},
           "runtime": {"num_ubatch": n_ub, "bwd_split": 1, "backend": "gloo", "timeout_s": 60, "placement": "split"},
           "train": {"deferred_batch_norm": False}}
    ref_losses, ref_teacher, ref_online = _ssl_oracle(n_steps, n_ub, 1)
    world = len(split_on) + len(split_tg)
    out = run_ranks(_ssl_rank, world, cfg, n_steps)
    losses = out[world - 1][0]                      # the loss rank is the last student rank
    assert len(losses) == n_steps
    torch.testing.assert_close(torch.tensor(losses), torch.tensor(ref_losses), rtol=2e-5, atol=1e-6)
    _, on, tg = out[0]
    got_t = [v for j in sorted(tg) for k, v in tg[j].items() if "running" not in k and "num_batches" not in k]
    want_t = list(ref_teacher.values())
    assert len(got_t) == len(want_t)
    for a, b in zip(got_t, want_t):
        torch.testing.assert_close(a, b, rtol=2e-5, atol=1e-6)
    got_o = [v for j in sorted(on) for k, v in on[j].items() if "running" not in k and "num_batches" not in k]
    want_o = [v for k, v in ref_online.items() if "running" not in k and "num_batches" not in k]
    assert len(got_o) == len(want_o)
    for a, b in zip(got_o, want_o):
        torch.testing.assert_close(a, b, rtol=2e-5, atol=1e-6)
