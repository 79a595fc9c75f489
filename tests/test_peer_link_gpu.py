"""Stage links over peer memory (copy engines + one-thread ordering kernels) between two GPUs: message order,
multi-tensor messages, channels-last tensors without a transpose, ring growth, flow control beyond the slot count,
and a bounded wait that reports instead of hanging when nothing is sent."""
import pytest
import torch

from tests.helpers import run_ranks

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _messages():
    g = torch.Generator().manual_seed(7)
    msgs = []
    for i in range(11):                       # more messages than slots; sizes grow at message 6
        n = 4 if i < 6 else 9
        a = torch.randn(n, 16, 6, 5, generator=g).to(torch.bfloat16)
        b = torch.randn(n, 33, generator=g)
        c = torch.tensor(float(i))
        msgs.append([a, b, c])
    return msgs


def _link_rank(rank, world):
    import os
    import time
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from tspipe_b200.comm.peer_link import LinkTimeout, PeerLink, make_link
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    store = dist.distributed_c10d._get_default_store()
    out = {}
    link = make_link(None, 1 - rank, dev, store=store, name="t/f0", peer_device=1 - rank, slots=3, limit_ms=20000,
                     channels_last=True)
    out["is_peer_link"] = isinstance(link, PeerLink)
    msgs = _messages()
    if rank == 0:
        for m in msgs:
            ts = [t.to(dev) for t in m]
            ts[0] = ts[0].contiguous(memory_format=torch.channels_last)
            link.send(ts)
        link.flush()
    else:
        # receives posted three ahead of their use, as the engine does
        handles, got = [], []
        for i, m in enumerate(msgs):
            handles.append(link.post_recv([(tuple(t.shape), t.dtype) for t in m]))
            if i >= 3:
                got.append(handles[i - 3].wait())
        for h in handles[-3:]:
            got.append(h.wait())
        torch.cuda.synchronize()
        out["equal"] = all(torch.equal(r.cpu(), t) for rs, m in zip(got, msgs) for r, t in zip(rs, m))
        out["channels_last_kept"] = all(rs[0].is_contiguous(memory_format=torch.channels_last) for rs in got)
        link.poll(sync=True)
    dist.barrier()
    # a receive that nothing answers: the wait gives up, the status says so, the context stays usable
    if rank == 1:
        quiet = PeerLink(store, "t/quiet", dev, slots=2, limit_ms=200)
        quiet._word = torch.zeros(8, dtype=torch.int32, device=dev)      # no sender exists: skip the rendezvous
        quiet._remote_word = (__import__("ctypes").c_void_p * 1)()
        quiet._remote_word[0] = quiet._word.data_ptr() + 16               # acknowledgements land in its own memory
        quiet._ring = torch.zeros(2 << 20, dtype=torch.uint8, device=dev)
        quiet._cap, quiet._epoch = 1 << 20, 1
        t0 = time.time()
        h = quiet.post_recv([((8,), torch.float32)])
        h.wait()
        torch.cuda.synchronize()
        out["wait_s"] = time.time() - t0
        try:
            quiet.poll(sync=True)
            out["raised"] = False
        except LinkTimeout:
            out["raised"] = True
        out["context_ok"] = float(torch.ones(64, device=dev).sum().item()) == 64.0
    dist.barrier()
    dist.destroy_process_group()
    return out


def test_peer_link_delivers_in_order_and_waits_are_bounded():
    out = run_ranks(_link_rank, 2, timeout=180)
    assert out[0]["is_peer_link"] and out[1]["is_peer_link"]
    assert out[1]["equal"] is True
    assert out[1]["channels_last_kept"] is True
    assert out[1]["raised"] is True and 0.15 <= out[1]["wait_s"] < 10.0
    assert out[1]["context_ok"] is True


def _pp2_rank(rank, world, peer_links, n_steps):
    import copy
    import torch.distributed as dist
    from torch import nn
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.models.mlp import mlp_sequential
    from tspipe_b200.optim import LARS
    torch.manual_seed(0)
    online = mlp_sequential([48, 64, 64, 32])
    target = copy.deepcopy(online)
    pred = nn.Sequential(nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 32))
    opt = LARS(list(online.parameters()) + list(pred.parameters()), lr=0.2, weight_decay=1e-4, momentum=0.9)
    n_on, n_tg = len(online) + len(pred), len(target)
    cfg = {"runtime": {"num_ubatch": 2, "bwd_split": 1, "dtype": "fp32", "timeout_s": 120, "peer_links": peer_links},
           "model_split": {"online": [2, n_on - 2], "target": [2, n_tg - 2]},
           "train": {"deferred_batch_norm": False}}
    tsp = TSPipe(online, target, pred, opt, byol_loss, ema_update, 0.9, "", config=cfg, device=f"cuda:{rank}")
    from tspipe_b200.comm.peer_link import PeerLink
    links = [l for l in (tsp.engine.fwd_in, tsp.engine.fwd_out, tsp.engine.bwd_in, tsp.engine.bwd_out) if l is not None]
    assert all(isinstance(l, PeerLink) == bool(peer_links) for l in links) and links
    g = torch.Generator().manual_seed(1)
    losses = []
    for _ in range(n_steps):
        a, b = torch.randn(32, 48, generator=g), torch.randn(32, 48, generator=g)
        l = tsp.feed(a.pin_memory(), b.pin_memory())
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    dist.destroy_process_group()
    return losses


def test_two_stage_pipeline_same_losses_over_peer_links_and_library_links():
    n_steps = 6
    peer = run_ranks(_pp2_rank, 2, True, n_steps)
    lib = run_ranks(_pp2_rank, 2, False, n_steps)
    a = [x for x in (peer[0] or peer[1])]
    b = [x for x in (lib[0] or lib[1])]
    assert len(a) == n_steps and len(b) == n_steps
    torch.testing.assert_close(torch.tensor(a), torch.tensor(b), rtol=1e-6, atol=1e-7)


def _split_ssl_rank(rank, world, n_steps):
    import torch.distributed as dist
    from tests.test_runtime_cpu import _ssl_batches, _ssl_models
    from tspipe_b200 import TSPipe
    from tspipe_b200.comm.peer_link import PeerLink
    from tspipe_b200.losses import byol_loss, ema_update
    online, target, predictor = _ssl_models()
    opt = torch.optim.SGD(list(online.parameters()) + list(predictor.parameters()), lr=0.1, momentum=0.9)
    cfg = {"model_split": {"online": [8], "target": [5]},
           "runtime": {"num_ubatch": 2, "bwd_split": 1, "dtype": "fp32", "timeout_s": 120, "placement": "split"},
           "train": {"deferred_batch_norm": False}}
    tsp = TSPipe(online, target, predictor, opt, byol_loss, ema_update, 0.9, "", config=cfg, device=f"cuda:{rank}")
    links = list(tsp.engine.ema_in.values()) + list(tsp.engine.ema_out.values())
    assert links and all(isinstance(l, PeerLink) for l in links)
    losses = []
    for i, (a, b) in enumerate(_ssl_batches(n_steps)):
        if i == 3:
            tsp.update_lr(0.05)
            tsp.update_momentum(0.95)
        l = tsp.feed(a.pin_memory(), b.pin_memory())
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    on, tg = tsp.state_dicts()
    dist.destroy_process_group()
    return losses, on, tg


def test_split_placement_momentum_teacher_on_two_gpus_matches_oracle():
    """Teacher on GPU 0, student on GPU 1: the student's parameters reach the teacher over a peer-memory link after
    every step, the teacher's outputs reach the loss through the peer-mapped ring; same numbers as the CPU oracle."""
    from tests.test_runtime_cpu import _ssl_oracle
    n_steps = 7
    ref_losses, ref_teacher, _ = _ssl_oracle(n_steps, 2, 1)
    out = run_ranks(_split_ssl_rank, 2, n_steps)
    torch.testing.assert_close(torch.tensor(out[1][0]), torch.tensor(ref_losses), rtol=2e-3, atol=1e-4)
    tg = out[0][2]
    got_t = [v for j in sorted(tg) for k, v in tg[j].items() if "running" not in k and "num_batches" not in k]
    for a, b in zip(got_t, list(ref_teacher.values())):
        torch.testing.assert_close(a, b, rtol=2e-3, atol=1e-4)
