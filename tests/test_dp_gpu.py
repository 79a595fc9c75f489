"""Two replicas as two processes on two GPUs: the peer-memory reduce-scatter + LARS + all-gather path
gives the same training trajectory as the NCCL all-reduce path and as the single-process oracle."""
import copy

import pytest
import torch
from torch import nn

from tests.helpers import run_ranks

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _models(dims=(48, 64, 64, 32)):
    from tspipe_b200.models.mlp import mlp_sequential
    torch.manual_seed(0)
    online = mlp_sequential(list(dims))
    target = copy.deepcopy(online)
    pred = nn.Sequential(nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 32))
    return online, target, pred


def _batches(n):
    g = torch.Generator().manual_seed(1)
    return [(torch.randn(32, 48, generator=g), torch.randn(32, 48, generator=g)) for _ in range(n)]


def _rank(rank, world, peer_memory, n_steps, dims=(48, 64, 64, 32)):
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.optim import LARS
    online, target, pred = _models(dims)
    opt = LARS(list(online.parameters()) + list(pred.parameters()), lr=0.2, weight_decay=1e-4, momentum=0.9)
    cfg = {"runtime": {"num_ubatch": 2, "bwd_split": 1, "dtype": "fp32", "dp_replicas": world, "timeout_s": 120,
                       "peer_memory": peer_memory},
           "model_split": {"online": [len(online) + len(pred)], "target": [len(target)]},
           "train": {"deferred_batch_norm": False}}
    tsp = TSPipe(online, target, pred, opt, byol_loss, ema_update, 0.9, "", config=cfg, device=f"cuda:{rank}")
    assert tsp.engine.dp_fused == bool(peer_memory)
    losses = []
    for a, b in _batches(n_steps):
        sl = slice(rank * 16, (rank + 1) * 16)
        l = tsp.feed(a[sl].pin_memory(), b[sl].pin_memory())
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    on, tg = tsp.state_dicts()
    dist.destroy_process_group()
    return losses, on, tg


@pytest.mark.parametrize("peer_memory,dims", [(True, (48, 64, 64, 32)), (False, (48, 64, 64, 32)),
                                              # odd tensor sizes: the 16-byte path of the peer kernels ends in scalar tails
                                              (True, (48, 63, 61, 32))])
def test_two_replicas_match_oracle(peer_memory, dims):
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.optim import LARS
    from tspipe_b200.oracle import DelayedTeacherOracle
    n_steps = 4
    online, target, pred = _models(dims)
    full = nn.Sequential(*list(online.children()), *list(pred.children()))
    opt = LARS(list(full.parameters()), lr=0.2, weight_decay=1e-4, momentum=0.9)
    orc = DelayedTeacherOracle(full, target, opt, byol_loss, ema_update, 0.9, kd=False, n_ubatch=4, bwd_split=1)
    n_t = len(list(target.parameters()))
    f = orc.update_fn
    orc.update_fn = lambda m, on, tg: f(m, on[:n_t], tg)
    ref = [orc.step(a, b) for a, b in _batches(n_steps)]
    out = run_ranks(_rank, 2, peer_memory, n_steps, dims)
    # each replica reports the loss of its half; their mean is the full-batch loss
    mean = [(x + y) / 2 for x, y in zip(out[0][0], out[1][0])]
    torch.testing.assert_close(torch.tensor(mean), torch.tensor(ref), rtol=2e-4, atol=1e-5)
    want = [v for k, v in full.state_dict().items()]
    got = [v for k, v in out[0][1][0].items()]
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b.detach(), rtol=1e-3, atol=1e-5)
