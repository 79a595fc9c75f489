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
