"""sm_100a kernels against plain PyTorch fp32 references of the same op."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def test_library_loads_and_exports():
    from tspipe_b200.ops import fused
    L = fused.lib()
    assert hasattr(L, "tsp_ema_update") and hasattr(L, "tsp_lars_step")


@pytest.mark.parametrize("n", [64, 4096 + 64, 1 << 20])
def test_ema_update(n):
    from tspipe_b200.ops import fused
    torch.manual_seed(0)
    t = torch.randn(n, device=_dev())
    s = torch.randn(n, device=_dev())
    want = t * 0.99 + s * 0.01
    shadow = torch.empty(n, dtype=torch.bfloat16, device=_dev())
    fused.ema_update_(t, s, 0.99, shadow)
    torch.testing.assert_close(t, want, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(shadow.float(), want, rtol=1e-2, atol=1e-2)


def _make_flat(shapes):
    from tspipe_b200.runtime.state import FlatParams
    ps = [torch.nn.Parameter(torch.randn(s, device=_dev())) for s in shapes]
    flat = FlatParams(ps, _dev(), with_grad=True)
    flat.grad.copy_(torch.randn_like(flat.grad))
    for i, p in enumerate(ps):       # padding must stay zero
        pass
    return ps, flat


SHAPES = [(64, 3, 7, 7), (64,), (64,), (256, 64, 1, 1), (1000, 333), (17,), (5, 5)]


@pytest.mark.parametrize("opt_name", ["lars", "adamw", "sgd"])
def test_flat_optimizers_match_per_tensor_reference(opt_name):
    from tspipe_b200.optim import LARS, SGD, AdamW
    import copy
    torch.manual_seed(1)
    ps, flat = _make_flat(SHAPES)
    ref_ps = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    mk = {"lars": lambda q: LARS(q, lr=0.3, weight_decay=1e-3, momentum=0.9),
          "adamw": lambda q: AdamW(q, lr=1e-2, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.05),
          "sgd": lambda q: SGD(q, lr=0.05, momentum=0.9, nesterov=True, weight_decay=1e-4)}[opt_name]
    opt, ref = mk(ps), mk(ref_ps)
    opt.bind_flat(flat, use_kernel=True)
    teacher = torch.randn(flat.total, device=_dev())
    ref_teacher = teacher.clone()
    opt.teacher_flat, opt.ema_momentum = teacher, 0.9
    for step in range(3):
        g = torch.randn_like(flat.grad)
        flat.grad.copy_(g)
        for i, (p, q) in enumerate(zip(ps, ref_ps)):
            q.grad = flat._view(flat.grad, i, p.data).detach().clone()
        opt.step()
        ref.step()
        for i, (p, q) in enumerate(zip(ps, ref_ps)):
            torch.testing.assert_close(p.detach(), q.detach(), rtol=2e-5, atol=2e-6)
            tv = flat._view(ref_teacher, i, p.data)
            tv.mul_(0.9).add_(q.detach(), alpha=0.1)
    for i, p in enumerate(ps):
        torch.testing.assert_close(flat._view(teacher, i, p.data), flat._view(ref_teacher, i, p.data),
                                   rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,d", [(1024, 256), (37, 100)])
def test_byol_loss(dtype, n, d):
    from tspipe_b200.losses import regression_loss
    from tspipe_b200.ops import fused
    torch.manual_seed(2)
    o1 = torch.randn(n, d, device=_dev(), dtype=dtype, requires_grad=True)
    o2 = torch.randn(n, d, device=_dev(), dtype=dtype, requires_grad=True)
    t1 = torch.randn(n, d, device=_dev(), dtype=dtype)
    t2 = torch.randn(n, d, device=_dev(), dtype=dtype)
    loss = fused.byol_loss(o1, o2, t1, t2)
    loss.backward()
    r1 = o1.detach().float().requires_grad_()
    r2 = o2.detach().float().requires_grad_()
    ref = (regression_loss(r1, t2.float()) + regression_loss(r2, t1.float())).mean()
    ref.backward()
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-4)
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(o1.grad.float(), r1.grad, **tol)
    torch.testing.assert_close(o2.grad.float(), r2.grad, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,c", [(64, 10), (256, 1000), (9, 30522)])
def test_kd_soft_target_loss(dtype, n, c):
    from tspipe_b200.ops import fused
    torch.manual_seed(3)
    s = (torch.randn(n, c, device=_dev()) * 2).to(dtype).requires_grad_()
    t = (torch.randn(n, c, device=_dev()) * 2).to(dtype)
    y = torch.randint(0, c, (n,), device=_dev())
    T, lambda_kd = 4.0, 0.7          # the reference's objective: CE + lambda_kd * T^2 * KL
    loss = fused.kd_soft_target_loss(s, t, y, T, 1.0, lambda_kd)
    loss.backward()
    r = s.detach().float().requires_grad_()
    ref = F.cross_entropy(r, y) + lambda_kd * T * T * F.kl_div(
        F.log_softmax(r / T, 1), F.softmax(t.float() / T, 1), reduction="batchmean")
    ref.backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=2e-4, atol=1e-5)
    tol = dict(rtol=1e-3, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-5)
    torch.testing.assert_close(s.grad.float(), r.grad, **tol)


def test_cross_entropy_with_ignored_rows():
    from tspipe_b200.ops import fused
    torch.manual_seed(4)
    s = torch.randn(50, 97, device=_dev(), requires_grad=True)
    y = torch.randint(0, 97, (50,), device=_dev())
    y[::3] = -100
    n_valid = int((y >= 0).sum())
    loss = fused.kd_ce_loss(s, None, y, 1.0, 1.0 / n_valid, 0.0)
    loss.backward()
    r = s.detach().clone().requires_grad_()
    ref = F.cross_entropy(r, y, ignore_index=-100)
    ref.backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s.grad, r.grad, rtol=1e-4, atol=1e-6)


def test_cosine_embedding_loss_masked():
    from tspipe_b200.ops import fused
    torch.manual_seed(5)
    x = torch.randn(40, 768, device=_dev(), requires_grad=True)
    y = torch.randn(40, 768, device=_dev())
    m = torch.rand(40, device=_dev()) > 0.3
    k = int(m.sum())
    loss = fused.cosine_embedding_loss(x, y, 1.0 / k, m)
    loss.backward()
    r = x.detach().clone().requires_grad_()
    ref = F.cosine_embedding_loss(r[m], y[m], torch.ones(k, device=_dev()))
    ref.backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(x.grad, r.grad, rtol=1e-3, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,d", [(197 * 4, 768), (33, 1024), (5, 64)])
def test_layer_norm(dtype, rows, d):
    from tspipe_b200.ops import fused
    torch.manual_seed(6)
    x = torch.randn(rows, d, device=_dev()).to(dtype).requires_grad_()
    w = torch.randn(d, device=_dev(), requires_grad=True)
    b = torch.randn(d, device=_dev(), requires_grad=True)
    g = torch.randn(rows, d, device=_dev()).to(dtype)
    y = fused.layer_norm(x, w, b, 1e-6)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr, br = w.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    yr = F.layer_norm(xr, (d,), wr, br, 1e-6)
    yr.backward(g.float())
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(y.float(), yr.detach(), **tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, **tol)
    wtol = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float32 else dict(rtol=5e-2, atol=0.3)
    torch.testing.assert_close(w.grad, wr.grad, **wtol)
    torch.testing.assert_close(b.grad, br.grad, **wtol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_bias(dtype):
    from tspipe_b200.ops import fused
    torch.manual_seed(7)
    x = torch.randn(64, 3072, device=_dev()).to(dtype).requires_grad_()
    b = torch.randn(3072, device=_dev(), requires_grad=True)
    g = torch.randn(64, 3072, device=_dev()).to(dtype)
    y = fused.gelu(x, b)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    brf = b.detach().clone().requires_grad_()
    yr = F.gelu(xr + brf)
    yr.backward(g.float())
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(y.float(), yr.detach(), **tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, **tol)
    torch.testing.assert_close(b.grad, brf.grad, rtol=2e-2, atol=0.2 if dtype == torch.bfloat16 else 1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,residual,relu", [((8, 64, 14, 14), True, True), ((4, 256, 7, 7), False, True),
                                                ((16, 24, 5, 3), False, False), ((32, 512), False, True),
                                                ((3, 2048, 2, 2), True, True),
                                                # >= 1 MB in bf16: the bulk-copy streaming statistics kernels
                                                ((64, 64, 28, 28), True, True), ((32, 256, 14, 14), False, True),
                                                ((16, 2048, 7, 7), True, True), ((48, 128, 9, 11), False, True),
                                                ((64, 64, 16, 16), False, False)])
def test_fused_batchnorm_act(dtype, shape, residual, relu):
    """Fused BN(+residual)(+ReLU) forward and backward vs. fp32 F.batch_norm + add + relu; the deferred
    accumulators must receive the microbatch sums."""
    from tspipe_b200.batchnorm import DeferredBatchNorm
    from tspipe_b200.ops import bn as fbn
    torch.manual_seed(8)
    c = shape[1]
    fmt = torch.channels_last if len(shape) == 4 else torch.contiguous_format
    x = (torch.randn(shape, device=_dev()) * 1.5 + 0.3).to(dtype).contiguous(memory_format=fmt).requires_grad_()
    res = torch.randn(shape, device=_dev()).to(dtype).contiguous(memory_format=fmt).requires_grad_() if residual else None
    g = torch.randn(shape, device=_dev()).to(dtype).contiguous(memory_format=fmt)
    bn = DeferredBatchNorm(c, chunks=3).to(_dev())
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.uniform_(-0.5, 0.5)
    assert fbn.applicable(bn, x)
    y = fbn.bn_act(bn, x, res, relu)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    rr = res.detach().float().requires_grad_() if residual else None
    wr, br = bn.weight.detach().clone().requires_grad_(), bn.bias.detach().clone().requires_grad_()
    yr = F.batch_norm(xr, None, None, wr, br, training=True, eps=bn.eps)
    if residual:
        yr = yr + rr
    # bf16: an element whose pre-activation is within rounding distance of zero may land on the other side of the
    # ReLU than in the fp32 reference, which flips its whole gradient; such elements are left out of the
    # element-wise comparison (their effect on the channel sums stays far below the tolerance)
    keep = torch.ones_like(yr, dtype=torch.bool)
    if relu:
        if dtype == torch.bfloat16:
            keep = yr.detach().abs() > 0.05
        yr = F.relu(yr)
    yr.backward(g.float())
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    assert keep.float().mean() > 0.9
    torch.testing.assert_close(y.float()[keep], yr.detach()[keep], **tol)
    torch.testing.assert_close(x.grad.float()[keep], xr.grad[keep], **tol)
    if residual:
        torch.testing.assert_close(res.grad.float()[keep], rr.grad[keep], **tol)
    wtol = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float32 else dict(rtol=5e-2, atol=0.5)
    torch.testing.assert_close(bn.weight.grad, wr.grad, **wtol)
    torch.testing.assert_close(bn.bias.grad, br.grad, **wtol)
    dims = [0] + list(range(2, len(shape)))
    xf = x.detach().float()
    torch.testing.assert_close(bn.sum, xf.sum(dims), rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(bn.sum_squares, (xf * xf).sum(dims), rtol=1e-3, atol=1e-2)
    assert bn.tracked == 1 and bn.counter == x.numel() // c
    assert fbn.stream_status() == 0


def test_fused_batchnorm_eval_uses_running_stats():
    from tspipe_b200.ops import bn as fbn
    torch.manual_seed(9)
    bn = torch.nn.BatchNorm2d(32).to(_dev())
    with torch.no_grad():
        bn.running_mean.normal_()
        bn.running_var.uniform_(0.5, 2.0)
    bn.eval()
    x = torch.randn(4, 32, 6, 6, device=_dev()).contiguous(memory_format=torch.channels_last)
    y = fbn.bn_act(bn, x, relu=True)
    torch.testing.assert_close(y, F.relu(bn(x)), rtol=1e-4, atol=1e-5)


def _two_gpus():
    return torch.cuda.device_count() >= 2


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ema_reads_student_from_peer_gpu():
    """The momentum update kernel running on cuda:0 reads the student buffer that lives on cuda:1."""
    from tspipe_b200.comm import peer
    from tspipe_b200.ops import fused
    torch.manual_seed(10)
    n = (1 << 20) + 64
    t = torch.randn(n, device="cuda:0")
    s = torch.randn(n, device="cuda:1")
    want = t.cpu() * 0.9 + s.cpu() * 0.1
    torch.cuda.synchronize("cuda:1")
    with torch.cuda.device(0):
        peer.enable_peer_access(1)
        fused.ema_update_(t, s, 0.9)
        torch.cuda.synchronize()
    torch.testing.assert_close(t.cpu(), want, rtol=1e-6, atol=1e-6)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("opt_name", ["lars", "adamw"])
def test_dp_fused_step_two_replicas_one_process(opt_name):
    """Two replicas emulated in one process (buffers on cuda:0 and cuda:1, peer access on): each rank's
    reduce-scatter + sharded step + all-gather kernels, run one after the other, must leave BOTH parameter
    buffers equal to the per-tensor reference optimizer stepped on the averaged gradient."""
    from tspipe_b200.comm import peer
    from tspipe_b200.comm.peer import pointer_table
    from tspipe_b200.ops import fused
    from tspipe_b200.optim import LARS, AdamW
    from tspipe_b200.runtime.state import FlatParams
    torch.manual_seed(11)
    devs = [torch.device("cuda", 0), torch.device("cuda", 1)]
    base = [torch.randn(s) for s in SHAPES]
    flats, states = [], []
    for d in devs:
        ps = [torch.nn.Parameter(b.clone().to(d)) for b in base]
        flats.append(FlatParams(ps, d, with_grad=True, pad_to=2))
    for i, d in enumerate(devs):
        with torch.cuda.device(d):
            peer.enable_peer_access(1 - i)
    ref_ps = [torch.nn.Parameter(b.clone()) for b in base]
    mk = {"lars": lambda q: LARS(q, lr=0.3, weight_decay=1e-3, momentum=0.9),
          "adamw": lambda q: AdamW(q, lr=1e-2, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.05)}[opt_name]
    ref = mk(ref_ps)
    total = flats[0].total
    shard = total // 2
    st = [{k: torch.zeros(total, device=d) for k in ("a", "b")} for d in devs]
    norms = [torch.zeros(2 * len(SHAPES), device=d) for d in devs]
    for step in range(1, 3):
        gs = [torch.randn(total) for _ in devs]
        for f, g in zip(flats, gs):
            f.grad.copy_(g.to(f.device))
        avg = (gs[0] + gs[1]) / 2
        for i, q in enumerate(ref_ps):
            q.grad = avg[flats[0].offsets[i]: flats[0].offsets[i] + flats[0].numels[i]].view(q.shape).clone()
        ref.step()
        torch.cuda.synchronize(0); torch.cuda.synchronize(1)
        rows_l = [[0.3, 1e-3, 0.9, 0.001, 1.0 if len(s) > 1 else 0.0] for s in SHAPES]
        rows_a = [[1e-2, 0.9, 0.98, 1e-6, 0.05, 1 - 0.9 ** step, 1 - 0.98 ** step] for _ in SHAPES]
        gptr = pointer_table([f.grad for f in flats])
        pptr = pointer_table([f.data for f in flats])
        if opt_name == "lars":
            for r, d in enumerate(devs):
                with torch.cuda.device(d):
                    hp = torch.tensor(rows_l, device=d)
                    ch = fused.build_chunks(flats[r].offsets, flats[r].numels, d, r * shard, (r + 1) * shard)
                    fused.dp_reduce_norms_(gptr, 2, 0.5, flats[r].grad, flats[r].data, ch, hp, norms[r])
                    torch.cuda.synchronize()
            tot = norms[0].cpu() + norms[1].cpu()            # the all-reduce of the partial norms
            for r, d in enumerate(devs):
                with torch.cuda.device(d):
                    hp = torch.tensor(rows_l, device=d)
                    ch = fused.build_chunks(flats[r].offsets, flats[r].numels, d, r * shard, (r + 1) * shard)
                    fused.dp_lars_apply_(pptr, 2, r, flats[r].grad, st[r]["a"], ch, hp, tot.to(d))
                    torch.cuda.synchronize()
        else:
            for r, d in enumerate(devs):
                with torch.cuda.device(d):
                    hp = torch.tensor(rows_a, device=d)
                    ch = fused.build_chunks(flats[r].offsets, flats[r].numels, d, r * shard, (r + 1) * shard)
                    fused.dp_adamw_step_(gptr, pptr, 2, r, 0.5, st[r]["a"], st[r]["b"], ch, hp)
                    torch.cuda.synchronize()
        for f in flats:
            for i, q in enumerate(ref_ps):
                got = f.data[f.offsets[i]: f.offsets[i] + f.numels[i]].view(q.shape).cpu()
                torch.testing.assert_close(got, q.detach(), rtol=3e-5, atol=3e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 64, 112, 112), (2, 16, 7, 9), (3, 8, 2, 2)])
def test_maxpool_channels_last(dtype, shape):
    from tspipe_b200.ops.pool import MaxPool3x3s2
    torch.manual_seed(12)
    x = torch.randn(shape, device=_dev()).to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_()
    pool = MaxPool3x3s2()
    y = pool(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = F.max_pool2d(xr, 3, 2, 1)
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr.detach(), rtol=0, atol=0)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("shape,residual", [((8, 64, 14, 14), True), ((64, 64, 28, 28), False), ((32, 256, 14, 14), True),
                                            ((16, 512), False)])
def test_batchnorm_stacked_views_match_separate_forwards(shape, residual):
    """Two views stacked along the batch axis under ``segments(2)`` = two separate fused forwards/backwards:
    per-view statistics, the same gradients, the same deferred running statistics."""
    import copy
    from tspipe_b200.batchnorm import BatchNormGroup, DeferredBatchNorm
    from tspipe_b200.ops import bn as fbn
    torch.manual_seed(11)
    c = shape[1]
    fmt = torch.channels_last if len(shape) == 4 else torch.contiguous_format
    mk = lambda s=1.0, o=0.0: (torch.randn(shape, device=_dev()) * s + o).bfloat16().contiguous(memory_format=fmt)
    xa, xb = mk(1.5, 0.3).requires_grad_(), mk(0.7, -1.0).requires_grad_()
    ra, rb = (mk().requires_grad_(), mk().requires_grad_()) if residual else (None, None)
    ga, gb = mk(), mk()
    net1 = torch.nn.Sequential(DeferredBatchNorm(c, chunks=1)).to(_dev())
    with torch.no_grad():
        net1[0].weight.uniform_(0.5, 1.5)
        net1[0].bias.uniform_(-0.5, 0.5)
    net2 = copy.deepcopy(net1)
    g1, g2 = BatchNormGroup(net1), BatchNormGroup(net2)
    # separate forwards
    ya = fbn.bn_act(net1[0], xa, ra, True)
    g1.step()
    yb = fbn.bn_act(net1[0], xb, rb, True)
    g1.step()
    torch.autograd.backward([ya, yb], [ga, gb])
    # stacked
    xs = torch.cat([xa.detach(), xb.detach()]).contiguous(memory_format=fmt).requires_grad_()
    rs = torch.cat([ra.detach(), rb.detach()]).contiguous(memory_format=fmt).requires_grad_() if residual else None
    with fbn.segments(2):
        ys = fbn.bn_act(net2[0], xs, rs, True)
    g2.step(2)
    ys.backward(torch.cat([ga, gb]))
    assert fbn.stream_status() == 0
    def close(got, want):
        # The per-channel sums are accumulated with atomics, so scale / shift differ in the last bit between the two
        # runs; an output that sits within rounding of zero may then fall on the other side of the ReLU, which flips
        # the gradient mask of that single element.  Allow a handful of such elements.
        bad = ((got.float() - want.float()).abs() > 2e-2 + 2e-2 * want.float().abs()).float().mean().item()
        assert bad < 1e-5, f"{bad:.2e} of the elements differ"
    close(ys, torch.cat([ya, yb]))
    close(xs.grad, torch.cat([xa.grad, xb.grad]))
    if residual:
        close(rs.grad, torch.cat([ra.grad, rb.grad]))
    for got, want in ((net2[0].weight.grad, net1[0].weight.grad), (net2[0].bias.grad, net1[0].bias.grad)):
        # one flipped ReLU element (see above) moves its channel's dw / db by about |dy * xhat| ~ 1
        off = ((got - want).abs() > 1e-2 + 1e-3 * want.abs())
        assert int(off.sum()) <= 2 and float((got - want).abs().max()) < 8.0, (int(off.sum()), float((got - want).abs().max()))
    torch.testing.assert_close(net2[0].running_mean, net1[0].running_mean, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(net2[0].running_var, net1[0].running_var, rtol=1e-4, atol=1e-5)
    assert int(net2[0].num_batches_tracked) == int(net1[0].num_batches_tracked) == 2


def test_mlm_head_vocab_padding_keeps_loss_and_gradients():
    """The MLM head pads a vocabulary that is no multiple of 8 with zero-probability classes on CUDA: the
    distillation loss and the gradients equal those of the unpadded logits."""
    from argparse import Namespace
    from tspipe_b200.losses import distil_loss
    from tspipe_b200.models.bert import BertConfig, MlmHead
    torch.manual_seed(12)
    cfg = BertConfig(vocab_size=130, hidden=32, layers=1, heads=4, ffn=64, max_pos=32, dropout=0.0)
    head_s, head_t = MlmHead(cfg).to(_dev()), MlmHead(cfg).to(_dev())
    x_s = torch.randn(4, 16, 32, device=_dev(), requires_grad=True)
    x_t = torch.randn(4, 16, 32, device=_dev())
    labels = torch.randint(0, 130, (4, 16), device=_dev())
    labels[:, ::3] = -100
    attn = torch.ones(4, 16, dtype=torch.long, device=_dev())
    extra = Namespace(temperature=2.0, alpha_ce=5.0, alpha_mlm=2.0, alpha_cos=1.0)
    s_out = head_s({"hidden": x_s})
    with torch.no_grad():
        t_out = head_t({"hidden": x_t})
    assert s_out[0].shape[-1] == 136 and t_out[0].shape[-1] == 136
    loss = distil_loss(s_out, t_out, (labels, attn), None, extra)
    loss.backward()
    # unpadded reference in fp32 PyTorch ops
    xr = x_s.detach().clone().requires_grad_()
    def plain(head, x):
        h = head.norm(F.gelu(F.linear(x, head.dense.weight, head.dense.bias)))
        return F.linear(h, head.decoder.weight, head.decoder.bias), x
    extra.no_fused = True
    ref = distil_loss(plain(head_s, xr), tuple(t.detach() for t in plain(head_t, x_t)), (labels, attn), None, extra)
    ref.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(x_s.grad, xr.grad, rtol=1e-2, atol=1e-4)


def test_multicast_capability_query_answers():
    """The NVLS capability probe is a driver attribute query: it answers True or False on a CUDA box and creates
    nothing."""
    from tspipe_b200.comm import peer
    before = torch.cuda.memory_allocated()
    ans = peer.multicast_supported(0)
    assert ans in (True, False)
    assert torch.cuda.memory_allocated() == before


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(8, 64, 7, 7), (3, 2048, 7, 7), (4, 24, 5, 3), (2, 512, 14, 14)])
def test_global_average_pool_matches_library(dtype, shape):
    """Channels-last global average pooling, forward and backward, against fp32 ``adaptive_avg_pool2d``."""
    from tspipe_b200.ops.pool import GlobalAvgPool, _GlobalAvgPool
    torch.manual_seed(5)
    x = torch.randn(shape, device=_dev()).to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_()
    g = torch.randn(shape[0], shape[1], 1, 1, device=_dev()).to(dtype)
    from tspipe_b200.ops import fused
    before = fused.LAUNCHES
    y = GlobalAvgPool()(x)
    y.backward(g)
    assert fused.LAUNCHES == before + 2                    # the kernels ran, not the fallback
    xr = x.detach().float().requires_grad_()
    yr = F.adaptive_avg_pool2d(xr, 1)
    yr.backward(g.float())
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    assert y.shape == yr.shape
    torch.testing.assert_close(y.float(), yr.detach(), **tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, **tol)
    assert x.grad.is_contiguous(memory_format=torch.channels_last)
