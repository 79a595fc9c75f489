"""Per-partition checkpoint files in the reference's format, and resuming from them."""
import os
import warnings

import torch
from torch import nn

from tests.helpers import run_ranks


def _loss(s, t, labels, args, extra, epoch):
    return torch.nn.functional.mse_loss(s, t) + torch.nn.functional.cross_entropy(s, labels)


def _models():
    torch.manual_seed(0)
    student = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 4))
    teacher = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 4))
    return student, teacher


def _batches():
    g = torch.Generator().manual_seed(5)
    return [(torch.randn(8, 8, generator=g), torch.randint(0, 4, (8,), generator=g)) for _ in range(6)]


def _rank(rank, world, art, first, last, resume):
    from tspipe_b200 import TSPipe, TSPipeMode
    student, teacher = _models()
    opt = torch.optim.SGD(student.parameters(), lr=0.1, momentum=0.9)
    cfg = {"model_split": {"online": [2, 3], "target": [1, 1]},
           "train": {"deferred_batch_norm": False, "save_model_every_iter": 3},
           "runtime": {"num_ubatch": 2, "bwd_split": 2, "backend": "gloo", "timeout_s": 60, "resume": resume}}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(student, teacher, None, opt, _loss, None, 1.0, art, config=cfg, device="cpu",
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False)
    for x, y in _batches()[first:last]:
        tsp.feed(x, x, y)
    tsp.stop()
    return tsp.state_dicts()[0]


def test_checkpoint_format_and_resume(tmp_path):
    a = str(tmp_path / "a")
    b = str(tmp_path / "b")
    full = run_ranks(_rank, 2, a, 0, 6, "")[0]
    run_ranks(_rank, 2, b, 0, 3, "")
    for part in (0, 1):
        blob = torch.load(os.path.join(b, f"model_batch3_part{part}.pt"), weights_only=False)
        assert {"online_network_state_dict", "target_network_state_dict", "optimizer_state_dict"} <= set(blob)
    assert set(torch.load(os.path.join(b, "model_batch3_part0.pt"), weights_only=False)["online_network_state_dict"]) \
        == {"0.weight", "0.bias"}                      # keys are the child names of the user's Sequential
    resumed = run_ranks(_rank, 2, str(tmp_path / "c"), 3, 6, b)[0]
    for j in full:
        for k in full[j]:
            torch.testing.assert_close(resumed[j][k], full[j][k], rtol=1e-5, atol=1e-6)


class _FakeEngine:
    """The attributes of an executor that the checkpoint code touches."""

    def __init__(self, online, target, optimizer):
        from tspipe_b200.batchnorm import BatchNormGroup
        self.online, self.target, self.optimizer = online, target, optimizer
        self.cuda, self.device, self.momentum, self.ga_count = False, torch.device("cpu"), 0.99, 0
        self.bn_group_online = BatchNormGroup(online)
        self.bn_group_target = BatchNormGroup(target)


def _flat_adamw(seed):
    from tspipe_b200.batchnorm import DeferredBatchNorm
    from tspipe_b200.optim import AdamW
    from tspipe_b200.runtime.state import FlatParams
    torch.manual_seed(seed)
    net = nn.Sequential(nn.Linear(8, 32), nn.BatchNorm1d(32), nn.ReLU(), nn.Linear(32, 4))
    net = DeferredBatchNorm.convert_deferred_batch_norm(net, chunks=4)
    tgt = nn.Sequential(nn.Linear(8, 4))
    opt = AdamW(net.parameters(), lr=1e-2)
    flat = FlatParams(list(net.parameters()), torch.device("cpu"), with_grad=True, pad_to=2)
    opt.bind_flat(flat, use_kernel=False)
    return net, tgt, opt, flat


def test_data_parallel_optimizer_shards_and_batchnorm_group_round_trip(tmp_path):
    """Replicas that each hold 1/R of the flat optimizer state write one range file each; loading reassembles
    the complete state on every replica.  The BatchNorm group's partly accumulated statistics come back too."""
    from tspipe_b200.ckpt import load_partition, save_partition
    art = str(tmp_path)
    full = None
    R = 2
    for r in range(R):
        net, tgt, opt, flat = _flat_adamw(0)
        flat.grad.copy_(torch.linspace(-1, 1, flat.total))
        opt.step()                                       # complete state (what a single replica would hold)
        if full is None:
            full = {k: v.clone() for k, v in opt._flat_state.items()}
        shard = flat.total // R
        for v in opt._flat_state.values():               # a replica's kernels only ever touch its own range
            v[: r * shard].zero_()
            v[(r + 1) * shard:].zero_()
        opt._dp, opt.handles_dp = {"r": R, "idx": r}, True
        eng = _FakeEngine(net, tgt, opt)
        eng.bn_group_online._acc.add_(1.5)
        eng.bn_group_online.tracked = 3
        save_partition(art, 7, 0, eng, replica=r)
    assert sorted(os.listdir(art)) == ["model_batch7_part0.pt", "model_batch7_part0_dp0.pt", "model_batch7_part0_dp1.pt"]
    net, tgt, opt, flat = _flat_adamw(1)
    eng = _FakeEngine(net, tgt, opt)
    sd_before = torch.load(os.path.join(art, "model_batch7_part0.pt"), weights_only=False)["optimizer_state_dict"]
    assert load_partition(art, 0, eng) == 7
    for k, v in full.items():
        torch.testing.assert_close(opt._flat_state[k], v)
    assert opt._steps == 1
    assert "tspipe_flat" in sd_before                      # loading leaves the caller's dict alone
    assert eng.bn_group_online.tracked == 3
    torch.testing.assert_close(eng.bn_group_online._acc, torch.full_like(eng.bn_group_online._acc, 1.5))
