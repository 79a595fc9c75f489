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


def _signal_rank(rank, world):
    """Phase 1 is signalled by both ranks; phase 2 is withheld by rank 1 until rank 0 has given up waiting."""
    import os
    import time
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from tspipe_b200.comm.signals import SignalPad
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    pad = SignalPad(dist.group.WORLD, [0, 1], rank, dev, limit_ms=5000)
    store = dist.distributed_c10d._get_default_store()
    out = {}
    data = torch.full((1024,), float(rank + 1), device=dev)
    pad.arrive(1)
    pad.wait(1)
    torch.cuda.synchronize()
    out["phase1_timed_out"] = pad.timed_out()
    if rank == 0:
        t0 = time.time()
        pad.wait(2, limit_ms=200)            # nobody sends phase 2 yet: the kernel gives up after 0.2 s
        torch.cuda.synchronize()
        out["wait_s"] = time.time() - t0
        out["phase2_timed_out"] = pad.timed_out()
        out["context_ok"] = float((data * 2).sum().item()) == 2048.0       # the stream and the context are intact
        store.set("gave_up", b"1")
        pad.arrive(2)
    else:
        store.wait(["gave_up"])              # the host withholds the signal until rank 0 has reported
        pad.arrive(2)
    pad.wait(2)                              # now both have arrived: the same wait completes
    torch.cuda.synchronize()
    out["phase2_late_timed_out"] = pad.timed_out()
    dist.barrier()
    dist.destroy_process_group()
    return out


def test_device_side_signal_wait_is_bounded():
    """A rank whose peer never sends a signal does not hang: the waiting kernel returns after its limit, the status
    word says so, the context stays usable, and once the peer does signal the same wait completes."""
    out = run_ranks(_signal_rank, 2, timeout=120)
    assert out[0]["phase1_timed_out"] is False and out[1]["phase1_timed_out"] is False
    assert out[0]["phase2_timed_out"] is True and 0.15 <= out[0]["wait_s"] < 5.0
    assert out[0]["context_ok"] is True
    assert out[0]["phase2_late_timed_out"] is False and out[1]["phase2_late_timed_out"] is False


def _adamw_resume_rank(rank, world, art, first, last, resume):
    """BYOL-style MLP job on two replicas with the fused data-parallel AdamW (optimizer state sharded over the
    replicas); checkpoints every 3 batches.  The target network is frozen: with a momentum teacher the look-ahead
    teacher forward of batch 4 has already run when the checkpoint of batch 3 is written, so a resumed run (which
    recomputes it from the newer teacher) legitimately differs from an uninterrupted one."""
    import warnings
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.optim import AdamW
    online, target, pred = _models()
    opt = AdamW(list(online.parameters()) + list(pred.parameters()), lr=1e-2, weight_decay=0.01)
    cfg = {"runtime": {"num_ubatch": 1, "bwd_split": 1, "dtype": "fp32", "dp_replicas": world, "timeout_s": 120,
                       "resume": resume},
           "model_split": {"online": [len(online) + len(pred)], "target": [len(target)]},
           "train": {"deferred_batch_norm": False, "save_model_every_iter": 3}}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(online, target, pred, opt, byol_loss, None, 1.0, art, config=cfg, device=f"cuda:{rank}")
    assert tsp.engine.dp_fused
    for a, b in _batches(6)[first:last]:
        sl = slice(rank * 16, (rank + 1) * 16)
        tsp.feed(a[sl].pin_memory(), b[sl].pin_memory())
    tsp.stop()
    on, tg = tsp.state_dicts()
    dist.destroy_process_group()
    return on


def test_resume_with_sharded_adamw_state_equals_uninterrupted_run(tmp_path):
    """Six steps in one go against three steps, a checkpoint (every replica writes its range of the optimizer state),
    and three more steps from it."""
    import os
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    full = run_ranks(_adamw_resume_rank, 2, a, 0, 6, "")[0]
    run_ranks(_adamw_resume_rank, 2, b, 0, 3, "")
    names = sorted(f for f in os.listdir(b) if f.startswith("model_batch3"))
    assert names == ["model_batch3_part0.pt", "model_batch3_part0_dp0.pt", "model_batch3_part0_dp1.pt"]
    resumed = run_ranks(_adamw_resume_rank, 2, c, 3, 6, b)[0]
    for k in full[0]:
        torch.testing.assert_close(resumed[0][k], full[0][k], rtol=1e-4, atol=1e-6)
