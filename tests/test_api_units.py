"""Small CPU tests of the public helper surface: config, batch_ops, splitter, optimizer re-binding, pytree,
affinity planning, data loaders, schedules, EMA plan."""
import copy

import pytest
import torch
from torch import nn

from tspipe_b200 import BalanceError, Batch, ScatterGatherFn, TSPipeModelOutput, TSPipeModelWrapper, gather, scatter
from tspipe_b200.affinity import AffinityManager
from tspipe_b200.batch_ops import BatchQueue, defaultScatterGatherFn
from tspipe_b200.config import DEFAULTS, load_yaml, merge_config, parse_cli
from tspipe_b200.dataloader import DummyInputGenerator, FastDataLoader
from tspipe_b200.runtime.ema_plan import build_ema_plans
from tspipe_b200.schedules import cosine_lr, cosine_momentum, linear_warmup_decay
from tspipe_b200.tspipe import default_balance, rebind_optimizer, split_module, verify_module
from tspipe_b200.utils import pytree as pt


def test_reference_yaml_loads_unchanged(tmp_path):
    p = tmp_path / "tspipe.yaml"
    p.write_text("""
tspipe:
  train:
    deferred_batch_norm: True
    save_model_every_iter: 100
  model_split:
    target: [2, 3, 2, 11]
    online: [2, 3, 2, 15]
  optimizer:
    skip_optimizer: False
    num_skip_initial_staleness: 0
    gradient_accumulation: 1
    reduce_verbose: False
  gpipe_emulation:
    enabled: False
    num_ubatch: 1
  async_param_update_emulation:
    enabled: False
""")
    cfg = load_yaml(str(p))
    assert cfg["model_split"]["online"] == [2, 3, 2, 15] and cfg["train"]["save_model_every_iter"] == 100
    assert cfg["runtime"] == DEFAULTS["runtime"]
    with pytest.raises(KeyError):
        merge_config({"optimizer": {"no_such_key": 1}})
    with pytest.raises(KeyError):
        merge_config({"nonsense": {}})


def test_cli_flags_coexist_with_application_flags():
    a = parse_cli(["--tspipe-config=x.yaml", "--ip=10.0.0.1", "--rank=1", "--num-nodes=2", "--app-flag", "7"])
    assert (a.tspipe_config, a.ip, a.rank, a.num_nodes) == ("x.yaml", "10.0.0.1", 1, 2)
    with pytest.raises(SystemExit):
        parse_cli(["--ip=x"], required=True)


def test_scatter_gather_roundtrip_and_errors():
    x = torch.arange(24.).view(6, 4)
    parts = scatter(x, 3)
    assert [p.tensor.shape[0] for p in parts] == [2, 2, 2] and parts[0].atomic
    torch.testing.assert_close(gather(parts), x)
    tup = (x, x * 2)
    tparts = scatter(tup, 2)
    g = gather(tparts)
    torch.testing.assert_close(g[1], x * 2)
    with pytest.raises(ValueError):
        scatter(torch.zeros(2, 3), 4)
    d = {"a": x, "n": 5, "m": None}
    dp = pt.generic_scatter(d, 3)
    assert dp[1]["n"] == 5 and dp[1]["a"].shape == (2, 4)
    torch.testing.assert_close(pt.generic_gather(dp)["a"], x)
    assert defaultScatterGatherFn.batch_size(x) == 6 and pt.leading_size(d) == 6


def test_batch_queue_ids_epochs_and_throttle():
    q = BatchQueue()
    assert q.get_new_batch_id() == 1 and q.get_new_batch_id() == 2
    assert q.wait_batch(2, timeout=0.01) and not q.wait_batch(3, timeout=0.01)
    q.report_epoch_boundary()
    assert q.epoch_boundaries == [2]
    q.stop()
    assert not q.wait_batch(5)


def test_split_module_balance_checks_and_predictor_names():
    online = nn.Sequential(nn.Linear(2, 2), nn.ReLU(), nn.Linear(2, 2))
    target = copy.deepcopy(online)
    pred = nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2))
    po, ptg = split_module(online, target, pred, [2, 3], [2, 1])
    assert [len(p) for p in po] == [2, 3] and [len(p) for p in ptg] == [2, 1]
    assert list(po[1].state_dict()) == ["2.weight", "2.bias", "predictor_0.weight", "predictor_0.bias",
                                        "predictor_1.weight", "predictor_1.bias"]
    with pytest.raises(BalanceError):
        split_module(online, target, pred, [2, 2], [2, 1])
    with pytest.raises(BalanceError):
        split_module(online, target, None, [3, 0], [2, 1])
    with pytest.raises(TypeError):
        verify_module(nn.Linear(1, 1))
    shared = nn.Linear(2, 2)
    with pytest.raises(ValueError):
        verify_module(nn.Sequential(shared, shared))
    assert default_balance(30, 4) == [8, 8, 7, 7]


def test_rebind_optimizer_keeps_group_hyperparameters():
    a, b = nn.Linear(2, 2), nn.Linear(2, 2)
    opt = torch.optim.SGD([{"params": a.parameters(), "lr": 0.1}, {"params": b.parameters(), "lr": 0.5}], lr=1.0)
    rebind_optimizer(opt, list(b.parameters()))
    assert [len(g["params"]) for g in opt.param_groups] == [0, 2]
    assert opt.param_groups[1]["lr"] == 0.5


def test_model_wrapper_passes_pytrees():
    class Two(nn.Module):
        def forward(self, d):
            return [d["x"] + 1, d["x"] * 2, None]
    w = TSPipeModelWrapper(Two())
    out = w({"x": torch.ones(2)})
    assert isinstance(out, TSPipeModelOutput) and out.data[2] is None
    out2 = TSPipeModelWrapper(nn.Identity())(TSPipeModelOutput({"x": 1}, None))
    assert isinstance(out2, TSPipeModelOutput)
    assert isinstance(TSPipeModelWrapper(nn.ReLU())(torch.ones(2)), torch.Tensor)
    leaves, spec, wrapped = pt.flatten(out)
    assert wrapped and len([l for l in leaves if isinstance(l, torch.Tensor)]) == 2
    assert isinstance(pt.unflatten(leaves, spec, wrapped), TSPipeModelOutput)


def test_affinity_plan_is_disjoint_and_prefers_local_cores():
    plan = AffinityManager.plan(3, allowed=list(range(16)), local=[{8, 9, 10, 11}, None, {0, 1}])
    assert plan[0] == [8, 9, 10, 11] and plan[2][:2] == [0, 1]
    flat = [c for p in plan for c in p]
    assert len(flat) == len(set(flat)) == 12

    class FakeNvml:
        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetCpuAffinity(self, h, n):
            return [0b1111 << (4 * h)] + [0] * (n - 1)
    assert AffinityManager.gpu_local_cores(1, nvml=FakeNvml()) == {4, 5, 6, 7}


def test_dummy_input_generator_and_fast_loader():
    gen = DummyInputGenerator(4, input_shape=8, length=3)
    items = list(gen)
    assert len(items) == 3 and items[0][0][0].shape == (4, 3, 8, 8) and items[0][0][0].is_shared()
    assert items[0][0][0] is items[2][0][0]
    ds = torch.utils.data.TensorDataset(torch.arange(10.))
    assert sum(len(b[0]) for b in FastDataLoader(ds, batch_size=4)) == 10


def test_schedules():
    assert cosine_lr(0, 100, 1.0, 10) == 0 and abs(cosine_lr(10, 100, 1.0, 10) - 1.0) < 1e-9
    assert cosine_lr(100, 100, 1.0, 10) < 1e-9
    assert cosine_momentum(0, 10, 0.99) == pytest.approx(0.99) and cosine_momentum(10, 10, 0.99) == pytest.approx(1.0)
    assert linear_warmup_decay(5, 100, 1.0, 10) == 0.5 and linear_warmup_decay(100, 100, 1.0, 10) == 0.0


def test_ema_plan_for_different_cuts():
    def net():
        return nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4), nn.Linear(4, 4), nn.Linear(4, 4))
    online, target = net(), net()
    po = [nn.Sequential(online[0]), nn.Sequential(online[1], online[2], online[3])]
    ptg = [nn.Sequential(target[0], target[1]), nn.Sequential(target[2], target[3])]
    plans = build_ema_plans(po, ptg)
    assert plans[0].local and 1 in plans[0].recv and 0 in plans[1].send and not plans[1].recv
    assert sum(n for _, _, n in plans[0].recv[1]) == sum(n for _, n in plans[1].send[0])
    same = build_ema_plans([nn.Sequential(online[0], online[1]), nn.Sequential(online[2], online[3])], ptg)
    assert all(p.is_local_prefix for p in same)
    bad = nn.Sequential(nn.Linear(4, 5))
    with pytest.raises(ValueError):
        build_ema_plans([bad], [nn.Sequential(target[0])])


def test_efficientnet_sequential_equals_module_and_logits_loss():
    from argparse import Namespace
    from tspipe_b200.losses import logits_kd
    from tspipe_b200.models.efficientnet import EfficientNet, drop_connect
    torch.manual_seed(0)
    net = EfficientNet("efficientnet-tiny-test", num_classes=7)
    assert net.test_sequential_validity((2, 3, 32, 32), rtol=1e-4, atol=1e-5)
    seq = net.to_sequential()
    assert len(seq) == 3 + len(net.blocks) + 3 + 4
    x = torch.ones(8, 2, 1, 1)
    assert drop_connect(x, 0.5, False) is x
    y = drop_connect(x, 0.5, True)
    assert set(y.flatten().tolist()) <= {0.0, 2.0}
    s, t = torch.randn(4, 7, requires_grad=True), torch.randn(4, 7)
    l = logits_kd(s, t, torch.tensor([0, 1, 2, 3]), extra_args=Namespace(lambda_kd=0.5))
    l.backward()
    assert s.grad is not None and l.item() > 0


def test_vit_convolution_stem_variant():
    """MoCo-v3's ``vit_conv_*`` models: 4 x (conv3x3/2 + BN + ReLU) + 1x1 projection as patch embedding, one
    transformer block fewer, default initialisation of the stem."""
    import torch
    from tspipe_b200.models.vit import CONFIGS, ConvStem, moco_vit_networks
    assert CONFIGS["vit_conv_base"].depth == 11 and CONFIGS["vit_conv_small"].depth == 11
    base, momentum, pred = moco_vit_networks("vit_conv_tiny_test", dim=16, mlp_dim=32)
    stem = next(iter(base.children()))
    assert isinstance(stem, ConvStem)
    convs = [m for m in stem.proj if isinstance(m, torch.nn.Conv2d)]
    assert [c.out_channels for c in convs] == [8, 16, 32, 64, 64] and convs[-1].kernel_size == (1, 1)
    assert all(torch.equal(a, b) for a, b in zip(base.state_dict().values(), momentum.state_dict().values()))
    x = torch.randn(4, 3, 32, 32)
    assert stem(x).shape == (4, 4, 64)
    assert pred(base(x)).shape == (4, 16)


def test_kd_losses_follow_the_reference_weighting():
    """``CE + lambda_kd * KD`` (`benchmarks/soft_target/train_kd.py:448-453`, ``--lambda_kd`` default 1.0);
    ``alpha`` selects the convex mix instead."""
    from argparse import Namespace
    import torch.nn.functional as F
    from tspipe_b200.losses import logits_kd, soft_target_kd
    torch.manual_seed(1)
    s, t, y = torch.randn(6, 5), torch.randn(6, 5), torch.randint(0, 5, (6,))
    T = 4.0
    ce = F.cross_entropy(s, y)
    kd = F.kl_div(F.log_softmax(s / T, 1), F.softmax(t / T, 1), reduction="batchmean") * T * T
    torch.testing.assert_close(soft_target_kd(s, t, y, extra_args=Namespace(T=T)), ce + kd)
    torch.testing.assert_close(soft_target_kd(s, t, y, extra_args=Namespace(T=T, lambda_kd=0.3)), ce + 0.3 * kd)
    torch.testing.assert_close(soft_target_kd(s, t, y, extra_args=Namespace(T=T, alpha=0.9)), 0.1 * ce + 0.9 * kd)
    torch.testing.assert_close(logits_kd(s, t, y, extra_args=Namespace(lambda_kd=2.0)), ce + 2.0 * F.mse_loss(s, t))
