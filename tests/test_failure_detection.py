"""Failure detection on the host (no GPU involved): a rank whose executor raises, and a rank that goes
silent, are reported to the other ranks, which fail fast instead of blocking."""
import pickle
import time
import warnings

import pytest
import torch
from torch import nn

from tests.helpers import run_ranks
from tspipe_b200.runtime.watchdog import PeerFailure, Watchdog


class FakeStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_watchdog_reports_death_notice_and_silence():
    store, now = FakeStore(), [100.0]
    failures = []
    w = Watchdog(store, 0, 3, heartbeat_s=1, timeout_s=5, progress=lambda: 7, on_failure=failures.append,
                 clock=lambda: now[0])
    w.beat()
    assert pickle.loads(store.get("hb/0")) == (100.0, 7, False)
    store.set("hb/1", pickle.dumps((99.9, 1)))
    store.set("hb/2", pickle.dumps((98.0, 1)))
    assert w.check_once() is None
    now[0] = 104.5
    f = w.check_once()
    assert isinstance(f, PeerFailure) and "rank 2" in str(f) and "silent" in str(f)
    store.set("bye/2", b"1")                      # a rank that left in an orderly way is not a failure
    store.set("hb/1", pickle.dumps((104.0, 2)))
    assert w.check_once() is None
    store.set("dead/1", b"ValueError('boom')")
    f = w.check_once()
    assert isinstance(f, PeerFailure) and "rank 1 failed" in str(f) and "boom" in str(f)


def test_watchdog_reports_rank_that_never_joined():
    store, now = FakeStore(), [0.0]
    w = Watchdog(store, 0, 2, 1, 3, lambda: 0, lambda e: None, clock=lambda: now[0])
    assert w.check_once() is None
    now[0] = 3.5
    assert "never reported" in str(w.check_once())


def _loss_that_fails(s, t, labels, args, extra, epoch):
    if int(labels[0]) == 99:
        raise ValueError("injected failure in the loss function")
    return torch.nn.functional.mse_loss(s, t)


def _rank(rank, world):
    from tspipe_b200 import TSPipe, TSPipeMode
    from tspipe_b200.runtime.engine import EngineError
    torch.manual_seed(0)
    student = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 8), nn.Linear(8, 4))
    teacher = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 4))
    opt = torch.optim.SGD(student.parameters(), lr=0.1)
    cfg = {"model_split": {"online": [2, 2], "target": [1, 1]},
           "runtime": {"num_ubatch": 2, "bwd_split": 1, "backend": "gloo", "timeout_s": 20, "heartbeat_s": 0.2},
           "train": {"deferred_batch_norm": False}}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        tsp = TSPipe(student, teacher, None, opt, _loss_that_fails, None, 1.0, "", config=cfg, device="cpu",
                     tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False)
    t0 = time.time()
    try:
        for i in range(50):
            x = torch.randn(4, 8)
            tsp.feed(x, x, torch.full((4,), 99 if i == 2 else 0))
            time.sleep(0.05)
        tsp.stop()
    except (EngineError, RuntimeError) as e:
        return "failed", time.time() - t0, str(e)[:300]
    return "finished", time.time() - t0, ""


def test_executor_exception_on_one_rank_stops_all_ranks():
    """The loss stage (rank 1) raises at batch 3; rank 0 learns about it from the store and raises from
    ``feed`` within a few heartbeats instead of blocking on its gradient receive."""
    out = run_ranks(_rank, 2, timeout=90, hard_exit=True)
    assert out[1][0] == "failed" and "injected failure" in out[1][2]
    assert out[0][0] == "failed" and ("rank 1 failed" in out[0][2] or "peer" in out[0][2])
    assert out[0][1] < 15 and out[1][1] < 15


def test_watchdog_reports_a_rank_that_beats_but_makes_no_progress():
    """A rank blocked inside a collective keeps its heartbeat thread alive: it is reported once it has stayed busy
    on the same operation count for the limit; an idle rank (waiting for input) with a constant count is not."""
    store, now = FakeStore(), [0.0]
    w = Watchdog(store, 0, 3, heartbeat_s=1, timeout_s=5, progress=lambda: 0, on_failure=lambda e: None,
                 clock=lambda: now[0], busy=lambda: True)
    w.beat()
    assert pickle.loads(store.get("hb/0")) == (0.0, 0, True)
    for t in (0.0, 2.0, 4.0, 6.0):
        now[0] = t
        store.set("hb/1", pickle.dumps((t, 11, True)))       # beating, busy, stuck on op 11
        store.set("hb/2", pickle.dumps((t, 4, False)))       # beating, idle
        f = w.check_once()
        if t <= 4.0:
            assert f is None
    assert isinstance(f, PeerFailure) and "rank 1 is stalled" in str(f) and "operation 11" in str(f)
    store.set("hb/1", pickle.dumps((6.0, 12, True)))         # progress resets the stall clock
    assert w.check_once() is None


@pytest.mark.gpu
def test_device_side_bounded_wait_gives_up_and_reports():
    """A kernel waits on an mbarrier that nothing completes (the signal is simply never sent).  The bounded wait of
    the tcgen05 kernels gives up after its limit, writes its code into the status word and the kernel returns: no
    trap, no hang, and the next kernel on the same context runs normally."""
    import ctypes as C
    from tspipe_b200.ops import conv, fused as f, gemm
    dev = torch.device("cuda", 0)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    L = conv._lib()
    L.tsp_bounded_wait_probe.restype = C.c_int
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.device(dev):
        e0.record()
        assert L.tsp_bounded_wait_probe(C.c_int(50), C.c_int(7), f._ptr(status), f._stream()) == 0
        e1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == 7
    assert 40.0 <= e0.elapsed_time(e1) <= 500.0
    # the context is intact: a tensor-core convolution right after gives the right answer
    x = torch.randn(2, 64, 8, 8, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    w = torch.randn(64, 64, 1, 1, device=dev) * 0.1
    y, _ = conv.conv2d(x, w)
    gemm.check_status()
    ref = torch.nn.functional.conv2d(x.float(), w.bfloat16().float())
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
