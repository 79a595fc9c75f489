"""Skip API: declaration checks, single-stage semantics, and a skip that crosses pipeline stages."""
import copy
from collections import OrderedDict

import pytest
import torch
from torch import nn

from tests.helpers import run_ranks
from tspipe_b200.skip import (Namespace, SkipSequential, inspect_skip_layout, pop, skippable, stash,
                              verify_skippables)


@skippable(stash=["res"])
class StashLinear(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.fc = nn.Linear(d, d)

    def forward(self, x):
        yield stash("res", x)
        return torch.relu(self.fc(x))


@skippable(pop=["res"])
class PopAdd(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.fc = nn.Linear(d, d)

    def forward(self, x):
        res = yield pop("res")
        return self.fc(x) + res


class Plain(nn.Module):
    """The same computation without the skip API."""

    def __init__(self, a, mid, b):
        super().__init__()
        self.a, self.mid, self.b = a, mid, b

    def forward(self, x):
        h = torch.relu(self.a.module.fc(x))
        for m in self.mid:
            h = m(h)
        return self.b.module.fc(h) + x


def _model(d=16):
    torch.manual_seed(0)
    return nn.Sequential(StashLinear(d), nn.Linear(d, d), nn.Tanh(), nn.Linear(d, d), PopAdd(d), nn.Linear(d, 8))


def test_verify_skippables_accepts_and_rejects():
    verify_skippables(_model())
    with pytest.raises(TypeError, match="not stashed"):
        verify_skippables(nn.Sequential(PopAdd(4)))
    with pytest.raises(TypeError, match="no module declared"):
        verify_skippables(nn.Sequential(StashLinear(4)))
    with pytest.raises(TypeError, match="not isolated"):
        verify_skippables(nn.Sequential(StashLinear(4), StashLinear(4), PopAdd(4), PopAdd(4)))
    ns1, ns2 = Namespace(), Namespace()
    verify_skippables(nn.Sequential(StashLinear(4).isolate(ns1), StashLinear(4).isolate(ns2),
                                    PopAdd(4).isolate(ns2), PopAdd(4).isolate(ns1)))


def test_single_partition_equals_plain_module():
    m = _model()
    seq = SkipSequential(OrderedDict(m.named_children()))
    x = torch.randn(5, 16, requires_grad=True)
    y = seq(x)
    plain = nn.Sequential(Plain(m[0], [m[1], m[2], m[3]], m[4]), m[5])
    x2 = x.detach().clone().requires_grad_()
    y2 = plain(x2)
    torch.testing.assert_close(y, y2)
    y.sum().backward()
    y2.sum().backward()
    torch.testing.assert_close(x.grad, x2.grad)


def test_layout_reports_cross_partition_routes():
    m = _model()
    parts = [nn.Sequential(m[0], m[1]), nn.Sequential(m[2], m[3]), nn.Sequential(m[4], m[5])]
    layout = inspect_skip_layout(parts)
    assert list(layout.copy_policy(2)) == [(0, None, "res")]
    assert layout.hops() == {0: [(None, "res")], 1: [(None, "res")]}


def _kd_loss(s, t, labels, args, extra, epoch):
    return torch.nn.functional.mse_loss(s, t) + torch.nn.functional.cross_entropy(s, labels)


def _rank(rank, world, n_steps):
    from tspipe_b200 import TSPipe, TSPipeMode
    student = _model()
    torch.manual_seed(1)
    teacher = nn.Sequential(nn.Linear(16, 16), nn.ReLU(), nn.Linear(16, 8))
    opt = torch.optim.SGD(student.parameters(), lr=0.1)
    cfg = {"model_split": {"online": [2, 2, 2], "target": [1, 1, 1]},
           "runtime": {"num_ubatch": 2, "bwd_split": 2, "backend": "gloo", "timeout_s": 60},
           "train": {"deferred_batch_norm": False}}
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(student, teacher, None, opt, _kd_loss, None, 1.0, "", tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM,
                     target_train_mode=False, config=cfg, device="cpu")
    g = torch.Generator().manual_seed(2)
    losses = []
    for _ in range(n_steps):
        x, y = torch.randn(8, 16, generator=g), torch.randint(0, 8, (8,), generator=g)
        l = tsp.feed(x, x, y)
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    return losses, tsp.state_dicts()[0]


def test_skip_crosses_two_stage_boundaries_in_pipeline():
    """The stash lives in stage 0 and the pop in stage 2: the skip tensor (and its gradient) ride over both
    links.  Result equals plain single-process training of the same model."""
    n_steps = 4
    student = _model()
    torch.manual_seed(1)
    teacher = nn.Sequential(nn.Linear(16, 16), nn.ReLU(), nn.Linear(16, 8))
    ref = SkipSequential(OrderedDict(student.named_children()))
    opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(2)
    want = []
    for _ in range(n_steps):
        x, y = torch.randn(8, 16, generator=g), torch.randint(0, 8, (8,), generator=g)
        with torch.no_grad():
            t = teacher(x)
        loss = _kd_loss(ref(x), t, y, None, None, 0)
        opt.zero_grad()
        loss.backward()
        opt.step()
        want.append(float(loss))
    out = run_ranks(_rank, 3, n_steps)
    torch.testing.assert_close(torch.tensor(out[2][0]), torch.tensor(want), rtol=1e-5, atol=1e-6)
    got = {}
    for st in out[0][1].values():
        got.update(st)
    for k, v in ref.state_dict().items():
        torch.testing.assert_close(got[k], v, rtol=1e-5, atol=1e-6)
