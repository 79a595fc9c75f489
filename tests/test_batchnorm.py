"""DeferredBatchNorm semantics (`tspipe/batchnorm.py:45-120`) and the flat statistics group."""
import copy

import torch
from torch import nn

from tspipe_b200.batchnorm import BatchNormGroup, DeferredBatchNorm


def _reference_deferred(bn: nn.BatchNorm2d, chunks):
    """Literal restatement of the reference layer: per-microbatch normalisation, extra sum / sum-of-squares
    reductions, commit with biased variance."""
    s = torch.zeros(bn.num_features)
    q = torch.zeros(bn.num_features)
    n = 0
    outs = []
    for x in chunks:
        s += x.sum((0, 2, 3))
        q += (x ** 2).sum((0, 2, 3))
        n += x.numel() // x.size(1)
        outs.append(torch.nn.functional.batch_norm(x, None, None, bn.weight, bn.bias, training=True, eps=bn.eps))
    mean = s / n
    var = q / n - mean ** 2
    rm = bn.running_mean * (1 - bn.momentum) + mean * bn.momentum
    rv = bn.running_var * (1 - bn.momentum) + var * bn.momentum
    return outs, rm, rv


def test_deferred_batchnorm_matches_reference_semantics():
    torch.manual_seed(0)
    bn = nn.BatchNorm2d(6)
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.normal_()
    x = torch.randn(12, 6, 5, 5) * 2 + 1
    chunks = list(x.chunk(3))
    want_outs, rm, rv = _reference_deferred(bn, chunks)
    d = DeferredBatchNorm.convert_deferred_batch_norm(nn.Sequential(copy.deepcopy(bn)), chunks=3)[0]
    for c, w in zip(chunks, want_outs):
        torch.testing.assert_close(d(c), w, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(d.running_mean, rm, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(d.running_var, rv, rtol=1e-4, atol=1e-5)
    assert int(d.num_batches_tracked) == 1 and d.tracked == 0
    d.eval()
    torch.testing.assert_close(d(x), torch.nn.functional.batch_norm(x, rm, rv, bn.weight, bn.bias, False, 0.0, bn.eps),
                               rtol=1e-5, atol=1e-5)


def test_converter_shares_parameters_and_buffers():
    m = nn.Sequential(nn.Conv2d(3, 4, 1), nn.BatchNorm2d(4), nn.Sequential(nn.BatchNorm2d(4)))
    w = m[1].weight
    c = DeferredBatchNorm.convert_deferred_batch_norm(m, chunks=2)
    assert isinstance(c[1], DeferredBatchNorm) and isinstance(c[2][0], DeferredBatchNorm)
    assert c[1].weight is w and c[1].chunks == 2
    assert set(c.state_dict()) >= {"1.running_mean", "1.sum", "1.sum_squares", "2.0.num_batches_tracked"}


def test_flat_group_equals_per_layer_commit():
    torch.manual_seed(1)
    def net():
        torch.manual_seed(2)
        return DeferredBatchNorm.convert_deferred_batch_norm(
            nn.Sequential(nn.Conv2d(3, 8, 3), nn.BatchNorm2d(8), nn.ReLU(), nn.Conv2d(8, 16, 3),
                          nn.BatchNorm2d(16, momentum=None), nn.Flatten(), nn.Linear(400, 4), nn.BatchNorm1d(4)), chunks=2)
    a, b = net(), net()
    x = torch.randn(8, 3, 9, 9)
    for m in list(a.modules()) + list(b.modules()):
        if isinstance(m, DeferredBatchNorm):
            m.sum.zero_(); m.sum_squares.zero_(); m.counter = 0; m.tracked = 0
            m.running_mean.zero_(); m.running_var.fill_(1); m.num_batches_tracked.zero_()
    group = BatchNormGroup(b)
    for rnd in range(2):
        for c in x.chunk(2):
            ya = a(c)
            yb = b(c)
            group.step()
            torch.testing.assert_close(ya, yb)
    sa, sb = a.state_dict(), b.state_dict()
    for k in sa:
        torch.testing.assert_close(sa[k].float(), sb[k].float(), rtol=1e-5, atol=1e-6, msg=k)
    assert int(sb["1.num_batches_tracked"]) == 2
