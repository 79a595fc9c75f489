"""Single-GPU engine checks: the CUDA path with the fused kernels equals the CPU oracle."""
import copy
import os

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


def test_smoke_entry():
    import __graft_entry__ as g
    g.smoke()


def test_single_gpu_byol_matches_oracle():
    """One stage on cuda:0, fp32, fused LARS + EMA + BYOL loss kernels, vs. the CPU oracle running
    the per-tensor LARS and the PyTorch loss."""
    os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29533")
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.models.mlp import mlp_sequential
    from tspipe_b200.optim import LARS
    from tspipe_b200.oracle import DelayedTeacherOracle
    import torch.distributed as dist

    def models():
        torch.manual_seed(0)
        online = mlp_sequential([48, 64, 64, 32], batch_norm=True)
        target = copy.deepcopy(online)
        pred = nn.Sequential(nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 32))
        return online, target, pred

    g = torch.Generator().manual_seed(1)
    batches = [(torch.randn(32, 48, generator=g), torch.randn(32, 48, generator=g)) for _ in range(5)]
    online, target, pred = models()
    full = nn.Sequential(*list(online.children()), *list(pred.children()))
    opt = LARS(list(full.parameters()), lr=0.2, weight_decay=1e-4, momentum=0.9)
    orc = DelayedTeacherOracle(full, target, opt, byol_loss, ema_update, 0.9, kd=False, n_ubatch=2, bwd_split=2)
    n_t = len(list(target.parameters()))
    f = orc.update_fn
    orc.update_fn = lambda m, on, tg: f(m, on[:n_t], tg)
    ref = [orc.step(a, b) for a, b in batches]

    online, target, pred = models()
    opt = LARS(list(online.parameters()) + list(pred.parameters()), lr=0.2, weight_decay=1e-4, momentum=0.9)
    cfg = {"runtime": {"num_ubatch": 2, "bwd_split": 2, "dtype": "fp32", "timeout_s": 120},
           "model_split": {"online": [len(online) + len(pred)], "target": [len(target)]},
           "train": {"deferred_batch_norm": False}}
    tsp = TSPipe(online, target, pred, opt, byol_loss, ema_update, 0.9, "", config=cfg, device="cuda:0")
    got = []
    for a, b in batches:
        l = tsp.feed(a.pin_memory(), b.pin_memory())
        if l is not None:
            got.append(l)
    got += tsp.stop()
    if dist.is_initialized():
        dist.destroy_process_group()
    torch.testing.assert_close(torch.tensor(got), torch.tensor(ref), rtol=2e-4, atol=1e-5)
    on_state, tg_state = tsp.state_dicts()
    want_t = list(orc.final_teacher().values())
    got_t = [v for k, v in tg_state[0].items() if "running" not in k and "num_batches" not in k]
    for a, b in zip(got_t, want_t):
        torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-5)


def _spawn_loss(o1, o2, t1, t2, args, extra):
    from tspipe_b200.losses import byol_loss
    return byol_loss(o1, o2, t1, t2)


def test_spawn_mode_worker_per_gpu(tmp_path):
    """The reference's launch style: one user process constructs TSPipe with the four CLI flags and the
    runtime spawns one worker process per visible GPU (here: all of them as pipeline stages)."""
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import ema_update
    from tspipe_b200.models.mlp import mlp_sequential
    from tspipe_b200.optim import LARS
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    if dist.is_initialized():
        dist.destroy_process_group()
    n = torch.cuda.device_count()
    torch.manual_seed(0)
    online = mlp_sequential([48, 64, 64, 32] + [32] * max(n - 1, 0), batch_norm=True)
    target = copy.deepcopy(online)
    pred = nn.Sequential(nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 32))
    opt = LARS(list(online.parameters()) + list(pred.parameters()), lr=0.2, weight_decay=1e-4)
    from tspipe_b200.tspipe import default_balance
    cfg = tmp_path / "t.yaml"
    cfg.write_text(f"""
tspipe:
  train: {{deferred_batch_norm: True, save_model_every_iter: 2}}
  model_split: {{online: {default_balance(len(online) + 3, n)}, target: {default_balance(len(target), n)}}}
  runtime: {{num_ubatch: 2, bwd_split: 1, dtype: fp32, timeout_s: 120}}
""")
    tsp = TSPipe(online, target, pred, opt, _spawn_loss, ema_update, 0.9, str(tmp_path),
                 argv=[f"--tspipe-config={cfg}", "--ip=127.0.0.1", "--rank=0", "--num-nodes=1"])
    g = torch.Generator().manual_seed(1)
    losses = []
    for _ in range(4):
        l = tsp.feed(torch.randn(16, 48, generator=g).share_memory_(), torch.randn(16, 48, generator=g).share_memory_())
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    assert len(losses) == 4 and all(l == l for l in losses)
    on, tg = tsp.state_dicts()
    assert len(on) == n and len(tg) == n
    assert (tmp_path / "model_batch2_part0.pt").exists()


def _kd_dict_job(cuda_graphs: bool):
    """Tiny BERT -> DistilBERT distillation on cuda:0 (dict stage inputs), losses of 6 steps."""
    import importlib.util
    from argparse import Namespace
    import torch.distributed as dist
    from tspipe_b200 import TSPipe, TSPipeMode
    from tspipe_b200.losses import distil_loss
    from tspipe_b200.models import bert as B
    from tspipe_b200.optim import AdamW
    spec = importlib.util.spec_from_file_location("dtrain", os.path.join(os.path.dirname(__file__), "..", "benchmarks",
                                                                         "distilbert", "train.py"))
    T = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(T)
    os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29534")
    torch.manual_seed(0)
    tcfg, scfg = B.BERT_TINY_TEST, B.DISTIL_TINY_TEST
    student, teacher = B.distillation_pair(tcfg, scfg)
    opt = AdamW(student.parameters(), lr=1e-3, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.0)
    cfg = {"runtime": {"num_ubatch": 1, "bwd_split": 1, "dtype": "bf16", "timeout_s": 120, "cuda_graphs": cuda_graphs},
           "model_split": {"online": [len(student)], "target": [len(teacher)]}, "train": {"deferred_batch_norm": False}}
    tsp = TSPipe(student, teacher, None, opt, distil_loss, None, 1.0, "", config=cfg, device="cuda:0",
                 tspipe_mode=TSPipeMode.SUPERVISED_MOMENTUM, target_train_mode=False, scatter_gather_fn=T.DICT_SG,
                 extra_args=Namespace(temperature=2.0, alpha_ce=5.0, alpha_mlm=2.0, alpha_cos=1.0))
    g = torch.Generator().manual_seed(0)
    losses = []
    for _ in range(6):
        ids = torch.randint(4, tcfg.vocab_size, (8, 16), generator=g)
        attn = torch.ones_like(ids)
        masked, labels = T.mask_tokens(ids, attn, tcfg.vocab_size, mask_id=3, generator=g)
        batch = {"input_ids": masked, "attention_mask": attn}
        l = tsp.feed(batch, batch, (labels, attn, int((labels >= 0).sum()), int(attn.sum())))
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    if dist.is_initialized():
        dist.destroy_process_group()
    return losses


def test_teacher_cuda_graph_with_dict_stage_inputs_matches_eager():
    """``runtime.cuda_graphs``: the frozen teacher's stage forward (a dict of tensors in, a tuple out) is replayed
    from a CUDA graph from the third batch on; the losses equal the eager run's."""
    eager = _kd_dict_job(False)
    graphed = _kd_dict_job(True)
    assert len(eager) == len(graphed) == 6
    torch.testing.assert_close(torch.tensor(graphed), torch.tensor(eager), rtol=2e-2, atol=2e-2)


def _byol_resnet_job(cuda_graphs: bool, ubatch: int, steps: int = 7):
    """BYOL on a ResNet-18 trunk at 64x64, bf16 + channels-last (the own convolution / BatchNorm kernels), one GPU."""
    import torch.distributed as dist
    from tspipe_b200 import TSPipe
    from tspipe_b200.losses import byol_loss, ema_update
    from tspipe_b200.models.resnet import byol_networks
    from tspipe_b200.optim import LARS
    from tspipe_b200.ops import fused
    os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29535")
    torch.manual_seed(0)
    online, target, pred = byol_networks("resnet18", 256, 64)
    opt = LARS(list(online.parameters()) + list(pred.parameters()), lr=0.05, weight_decay=1e-6, momentum=0.9)
    cfg = {"runtime": {"num_ubatch": ubatch, "bwd_split": 1, "dtype": "bf16", "channels_last": True, "timeout_s": 120,
                       "cuda_graphs": cuda_graphs},
           "model_split": {"online": [len(online) + len(pred)], "target": [len(target)]},
           "train": {"deferred_batch_norm": True}}
    tsp = TSPipe(online, target, pred, opt, byol_loss, ema_update, 0.99, "", config=cfg, device="cuda:0")
    g = torch.Generator().manual_seed(3)
    losses, launches = [], []
    for _ in range(steps):
        a, b = torch.randn(32, 3, 64, 64, generator=g), torch.randn(32, 3, 64, 64, generator=g)
        n0 = fused.LAUNCHES
        l = tsp.feed(a.pin_memory(), b.pin_memory())
        if l is not None:
            losses.append(l)
    losses += tsp.stop()
    on, _ = tsp.state_dicts()
    slots = tsp.engine.student_graphs.slots if tsp.engine.student_graphs is not None else {}
    captured = sum(1 for s in slots.values() if s.fwd is not None)
    if dist.is_initialized():
        dist.destroy_process_group()
    return losses, on, captured


@pytest.mark.parametrize("ubatch", [1, 2])
def test_student_stage_cuda_graphs_match_eager(ubatch):
    """``runtime.cuda_graphs``: after two eager calls per microbatch slot the student stage's forward and backward are
    replayed from CUDA graphs (weights cast inside the graph, gradients added to the flat buffer inside the graph);
    the losses and the trained weights are those of the eager run up to the noise of the atomically summed weight
    gradients."""
    eager, w_eager, n0 = _byol_resnet_job(False, ubatch)
    again, w_again, _ = _byol_resnet_job(False, ubatch)          # the run-to-run noise of the eager path itself
    graphed, w_graph, n1 = _byol_resnet_job(True, ubatch)
    assert n0 == 0 and n1 == ubatch
    assert len(eager) == len(graphed) == 7
    torch.testing.assert_close(torch.tensor(graphed), torch.tensor(eager), rtol=2e-2, atol=2e-2)

    def distance(x, y):
        num = sum(float((x[0][k].float() - y[0][k].float()).pow(2).sum()) for k in y[0] if y[0][k].is_floating_point())
        den = sum(float(y[0][k].float().pow(2).sum()) for k in y[0] if y[0][k].is_floating_point())
        return (num / den) ** 0.5
    noise = distance(w_again, w_eager)
    assert distance(w_graph, w_eager) <= 3.0 * noise + 2e-3, (distance(w_graph, w_eager), noise)
