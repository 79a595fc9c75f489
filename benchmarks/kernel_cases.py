"""Small stand-alone cases of the hand-written kernels, for profiling one kernel at a time.

    python benchmarks/kernel_cases.py bn        # fused BatchNorm fwd/bwd on one ResNet-50 activation
    python benchmarks/kernel_cases.py bn_r50    # all 53 BatchNorm layers of ResNet-50, forward + backward
    python benchmarks/kernel_cases.py stem      # tcgen05 stem convolution 7x7/2 on [128, 3, 224, 224]
    python benchmarks/kernel_cases.py lars      # flat LARS + fused EMA step over 25 M parameters
    python benchmarks/kernel_cases.py ema       # momentum-teacher update over 25 M parameters
    python benchmarks/kernel_cases.py kd        # soft-target KD loss on [2048, 1000] logits
    python benchmarks/kernel_cases.py ln        # LayerNorm fwd/bwd on [512*197, 768]
    python benchmarks/kernel_cases.py gemm [M N K]   # tcgen05 GEMM (default 8192 x 3072 x 768)
    python benchmarks/kernel_cases.py infonce   # MoCo InfoNCE forward + backward, 4096 x 256
    python benchmarks/kernel_cases.py attn      # ViT-B attention forward (tcgen05 flash-style kernel)
    python benchmarks/kernel_cases.py conv [N]  # every 1x1 / 3x3 convolution shape of ResNet-50 (batch N, default 256):
                                                # implicit-GEMM forward / data grad / weight grad against the library
    python benchmarks/kernel_cases.py conv1 CIN COUT K STRIDE SIDE [N]   # one convolution shape (profiling)

Each case allocates a few hundred MB at most (inputs larger than the 126 MB L2 where DRAM figures
matter), runs the op a handful of times and prints CUDA-event timings with the achieved bandwidth.
"""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _time(fn, n=5, flush=None):
    fn()
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(n):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best * 1e3


def case_bn():
    from tspipe_b200.batchnorm import DeferredBatchNorm
    from tspipe_b200.ops import bn as fbn
    dev = torch.device("cuda")
    shp = (128, 64, 112, 112)
    x = torch.randn(shp, device=dev).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_()
    g = torch.randn(shp, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
    bn = DeferredBatchNorm(64, chunks=10 ** 9).to(dev)
    nbytes = x.numel() * 2
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tf = _time(lambda: fbn.bn_act(bn, x, None, True), flush=flush)
    y = fbn.bn_act(bn, x, None, True)
    tb = _time(lambda: torch.autograd.grad(y, x, g, retain_graph=True), flush=flush)
    print(f"bn fwd  {shp}: {tf:8.1f} us  {3 * nbytes / tf / 1e6:5.2f} TB/s (read x twice, write y)")
    print(f"bn bwd  {shp}: {tb:8.1f} us  {5 * nbytes / tb / 1e6:5.2f} TB/s (read dy,x twice, write dx)")


# BatchNorm inputs of ResNet-50 at 224 x 224 (channels, side, residual?, count): stem, then per stage the three
# normalisations of each bottleneck (+ the downsample one)
R50_BN = [(64, 112, False, 1)] + \
    [(64, 56, False, 6), (256, 56, True, 3), (256, 56, False, 1)] + \
    [(128, 56, False, 1), (128, 28, False, 7), (512, 28, True, 4), (512, 28, False, 1)] + \
    [(256, 28, False, 1), (256, 14, False, 11), (1024, 14, True, 6), (1024, 14, False, 1)] + \
    [(512, 14, False, 1), (512, 7, False, 5), (2048, 7, True, 3), (2048, 7, False, 1)]


def case_bn_r50():
    """Every BatchNorm of one ResNet-50 forward + backward at batch 128 (no L2 flush between layers, as in
    the model): fused statistics + apply kernels against ATen batch_norm (+ add + relu)."""
    import torch.nn.functional as F
    from tspipe_b200.batchnorm import DeferredBatchNorm
    from tspipe_b200.ops import bn as fbn
    dev = torch.device("cuda")
    layers = []
    total = 0
    for c, side, res, count in R50_BN:
        shp = (128, c, side, side)
        x = torch.randn(shp, device=dev).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_()
        r = torch.randn_like(x) if res else None
        bn = DeferredBatchNorm(c, chunks=10 ** 9).to(dev)
        layers.append((bn, x, r, torch.randn_like(x), count))
        total += x.numel() * 2 * count

    def ours(backward):
        for bn, x, r, g, count in layers:
            for _ in range(count):
                y = fbn.bn_act(bn, x, r, True)
                if backward:
                    torch.autograd.grad(y, x, g)

    def aten(backward):
        for bn, x, r, g, count in layers:
            for _ in range(count):
                y = F.batch_norm(x, None, None, bn.weight.bfloat16(), bn.bias.bfloat16(), True)
                y = F.relu(y + r if r is not None else y)
                if backward:
                    torch.autograd.grad(y, x, g)

    for name, fn in (("fused kernels", ours), ("ATen", aten)):
        tf = _time(lambda: fn(False), n=3)
        tfb = _time(lambda: fn(True), n=3)
        print(f"R50 BatchNorm x53, batch 128, {total / 1e9:.2f} GB of activations, {name:14s}: "
              f"forward {tf / 1e3:6.2f} ms   forward+backward {tfb / 1e3:6.2f} ms")
    print("streaming-kernel status:", fbn.stream_status())


def case_stem():
    """ResNet stem convolution [128, 3, 224, 224] -> [128, 64, 112, 112] (+ BatchNorm statistics) against the
    library convolution followed by the statistics kernel."""
    import torch.nn.functional as F
    from tspipe_b200.ops import conv, gemm
    dev = torch.device("cuda")
    x = torch.randn(128, 3, 224, 224, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    w = torch.randn(64, 3, 7, 7, device=dev) * 0.05
    wb = w.bfloat16().contiguous(memory_format=torch.channels_last)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    torch.backends.cudnn.benchmark = True
    t = _time(lambda: conv.stem_conv(x, w), n=10, flush=flush)
    tr = _time(lambda: F.conv2d(x, wb, stride=2, padding=3), n=10, flush=flush)
    gemm.check_status()
    out_bytes = 128 * 64 * 112 * 112 * 2
    flops = 2 * 128 * 112 * 112 * 64 * 147
    print(f"stem conv 7x7/2 [128,3,224,224]: {t:8.1f} us  ({(out_bytes + x.numel() * 2) / t / 1e6:5.2f} TB/s, "
          f"{flops / t / 1e6:6.1f} TFLOP/s)   library: {tr:8.1f} us")


def case_lars():
    from tspipe_b200.optim import LARS
    from tspipe_b200.runtime.state import FlatParams
    dev = torch.device("cuda")
    ps = [torch.nn.Parameter(torch.randn(2048, 1024, device=dev)) for _ in range(12)] + \
         [torch.nn.Parameter(torch.randn(2048, device=dev)) for _ in range(12)]
    flat = FlatParams(ps, dev, with_grad=True)
    flat.grad.normal_()
    opt = LARS(ps, lr=0.1, weight_decay=1e-6)
    opt.bind_flat(flat, use_kernel=True)
    opt.teacher_flat, opt.ema_momentum = torch.randn(flat.total, device=dev), 0.996
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    t = _time(opt.step, flush=flush)
    n = flat.total
    print(f"lars+ema step over {n / 1e6:.1f} M params: {t:8.1f} us  {n * 4 * 9 / t / 1e6:5.2f} TB/s "
          "(norms: read p,g; apply: read p,g,mu,t write p,mu,t)")


def case_ema():
    from tspipe_b200.ops import fused
    dev = torch.device("cuda")
    n = 64 << 20
    t_, s_ = torch.randn(n, device=dev), torch.randn(n, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    t = _time(lambda: fused.ema_update_(t_, s_, 0.996), flush=flush)
    print(f"ema over {n / 1e6:.0f} M params: {t:8.1f} us  {n * 12 / t / 1e6:5.2f} TB/s")


def case_kd():
    from tspipe_b200.ops import fused
    dev = torch.device("cuda")
    s = torch.randn(2048, 1000, device=dev).bfloat16().requires_grad_()
    tt = torch.randn(2048, 1000, device=dev).bfloat16()
    y = torch.randint(0, 1000, (2048,), device=dev)
    t = _time(lambda: fused.kd_soft_target_loss(s, tt, y, 4.0, 1.0, 1.0))
    print(f"kd loss [2048,1000] fwd+grad: {t:8.1f} us")


def case_ln():
    from tspipe_b200.ops import fused
    dev = torch.device("cuda")
    rows, d = 512 * 197, 768
    x = torch.randn(rows, d, device=dev).bfloat16().requires_grad_()
    w = torch.ones(d, device=dev, requires_grad=True)
    b = torch.zeros(d, device=dev, requires_grad=True)
    g = torch.randn(rows, d, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tf = _time(lambda: fused.layer_norm(x, w, b, 1e-6), flush=flush)
    y = fused.layer_norm(x, w, b, 1e-6)
    tb = _time(lambda: torch.autograd.grad(y, (x, w, b), g, retain_graph=True), flush=flush)
    nb = rows * d * 2
    print(f"layernorm fwd [{rows},{d}]: {tf:8.1f} us  {2 * nb / tf / 1e6:5.2f} TB/s")
    print(f"layernorm bwd [{rows},{d}]: {tb:8.1f} us  {3 * nb / tb / 1e6:5.2f} TB/s")


def case_gemm():
    from tspipe_b200.ops import gemm
    dev = torch.device("cuda")
    m, n, k = (int(v) for v in sys.argv[2:5]) if len(sys.argv) > 4 else (8192, 3072, 768)
    a = torch.randn(m, k, device=dev).bfloat16()
    b = torch.randn(n, k, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bias = torch.randn(n, device=dev)
    t2 = _time(lambda: gemm.matmul_nt(a, b, two_cta=True), n=10, flush=flush)
    t2b = _time(lambda: gemm.matmul_nt(a, b, bias, two_cta=True), n=10, flush=flush)
    t1 = _time(lambda: gemm.matmul_nt(a, b, two_cta=False), n=10, flush=flush)
    tr = _time(lambda: a @ b.t(), n=10, flush=flush)
    gemm.check_status()
    f = 2 * m * n * k / 1e6
    print(f"tcgen05 gemm {m}x{n}x{k}: CTA pair {t2:7.1f} us {f / t2:7.1f} TFLOP/s (with bias {t2b:7.1f} us) | one CTA {t1:7.1f} us {f / t1:7.1f} TFLOP/s"
          f" | library {tr:7.1f} us {f / tr:7.1f} TFLOP/s")


def case_infonce():
    import torch.nn.functional as F
    from tspipe_b200.ops import fused, gemm
    dev = torch.device("cuda")
    n, d, temp = (int(sys.argv[2]) if len(sys.argv) > 2 else 4096), 256, 0.2
    q = torch.randn(n, d, device=dev, requires_grad=True)
    k = torch.randn(n, d, device=dev)

    def ours():
        q.grad = None
        fused.info_nce_loss(q, k, temp).backward()

    def ref():
        q.grad = None
        logits = F.normalize(q, dim=1) @ F.normalize(k, dim=1).t() / temp
        (F.cross_entropy(logits, torch.arange(n, device=dev)) * 2 * temp).backward()

    def device_time(fn):
        """Device time of one call with the launch overhead taken out: the call is captured into a CUDA graph and
        the replays are timed (a dozen small launches per call would otherwise be bound by the host)."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return _time(g.replay, n=10)

    t = device_time(ours)
    gemm.set_nce_key_split(False)
    t1 = device_time(ours)
    gemm.set_nce_key_split(True)
    gemm.set_fused_nce(False)
    tu = device_time(ours)
    gemm.set_fused_nce(True)
    tr = device_time(ref)
    gemm.check_status()
    flops = 2 * 2 * n * n * d          # scores + weighted sum of keys
    print(f"info_nce fwd+bwd [{n},{d}] (graph replays, device time): fused kernel with the keys split over "
          f"{gemm.nce_key_chunks(n, n)} chunks {t:7.1f} us ({flops / t / 1e6:6.1f} TFLOP/s incl. normalisation and merge "
          f"kernels) | one CTA per query tile {t1:7.1f} us | logits GEMM + CE kernel {tu:7.1f} us | library ops "
          f"{tr:7.1f} us")


def case_attn():
    """ViT-B attention forward, batch 256 x 12 heads x 197 tokens x 64: tcgen05 kernel against the library."""
    import torch.nn.functional as F
    from tspipe_b200.ops import attention, gemm
    dev = torch.device("cuda")
    b, h, n, dh = 256, 12, 197, 64
    qkv = torch.randn(b, n, 3, h, dh, device=dev).bfloat16()
    q, k, v = qkv.permute(2, 0, 3, 1, 4)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    with torch.no_grad():
        t = _time(lambda: attention.flash_fwd(q, k, v), n=10, flush=flush)
        tr = _time(lambda: F.scaled_dot_product_attention(q, k, v), n=10, flush=flush)
    gemm.check_status()
    flops = 4 * b * h * n * n * dh
    byts = 4 * b * h * n * dh * 2
    print(f"attention fwd [{b},{h},{n},{dh}]: {t:7.1f} us ({flops / t / 1e6:6.1f} TFLOP/s, {byts / t / 1e6:5.2f} TB/s) | "
          f"library {tr:7.1f} us")


# 1x1 / 3x3 convolutions of ResNet-50 at 224 x 224: (cin, cout, kernel, stride, input side, how many)
R50_CONV = [(64, 64, 1, 1, 56, 1), (64, 64, 3, 1, 56, 3), (64, 256, 1, 1, 56, 4), (256, 64, 1, 1, 56, 2),
            (256, 128, 1, 1, 56, 1), (128, 128, 3, 2, 56, 1), (128, 512, 1, 1, 28, 4), (256, 512, 1, 2, 56, 1),
            (512, 128, 1, 1, 28, 3), (128, 128, 3, 1, 28, 3),
            (512, 256, 1, 1, 28, 1), (256, 256, 3, 2, 28, 1), (256, 1024, 1, 1, 14, 6), (512, 1024, 1, 2, 28, 1),
            (1024, 256, 1, 1, 14, 5), (256, 256, 3, 1, 14, 5),
            (1024, 512, 1, 1, 14, 1), (512, 512, 3, 2, 14, 1), (512, 2048, 1, 1, 7, 3), (1024, 2048, 1, 2, 14, 1),
            (2048, 512, 1, 1, 7, 2), (512, 512, 3, 1, 7, 2)]


def _conv_one(cin, cout, k, stride, side, n, flush):
    """(own fprop, own dgrad, own wgrad, library fprop, library dgrad + wgrad) in microseconds, and the FLOPs of one
    of the three products."""
    import torch.nn.functional as F
    from tspipe_b200.ops import conv, gemm
    dev = torch.device("cuda")
    pad = (k - 1) // 2
    x = torch.randn(n, cin, side, side, device=dev).to(dtype=torch.bfloat16, memory_format=torch.channels_last)
    wgt = (torch.randn(cout, cin, k, k, device=dev) * 0.05).to(memory_format=torch.channels_last)
    w16 = wgt.to(torch.bfloat16)
    xg = x.clone().requires_grad_()
    wp = wgt.clone().requires_grad_()
    y, _ = conv.conv2d(xg, wp, stride, want_sums=True, segments=2)
    g = torch.randn_like(y)
    so = side // stride
    flops = 2.0 * n * so * so * cout * cin * k * k
    t_f = _time(lambda: conv.conv2d(x, wgt, stride, want_sums=True, segments=2), flush=flush)
    L = conv._lib()
    import ctypes as C
    from tspipe_b200.ops import fused as f
    st = f._ptr(gemm._status_word(dev))
    dx = torch.empty_like(x)
    dw = torch.zeros(cout, k, k, cin, device=dev)
    w16k = conv._w16(wgt)
    args = (C.c_int(n), C.c_int(side), C.c_int(side), C.c_int(cin), C.c_int(cout), C.c_int(k), C.c_int(stride))
    t_d = _time(lambda: L.tsp_conv_dgrad(f._ptr(g), f._ptr(w16k), f._ptr(dx), *args, st, f._stream()), flush=flush)
    t_w = _time(lambda: L.tsp_conv_wgrad(f._ptr(x), f._ptr(g), f._ptr(dw), *args, st, f._stream()), flush=flush)
    gemm.check_status()
    t_lf = _time(lambda: F.conv2d(x, w16, stride=stride, padding=pad), flush=flush)
    t_lb = _time(lambda: torch.ops.aten.convolution_backward(g, x, w16, None, [stride, stride], [pad, pad], [1, 1], False,
                                                             [0, 0], 1, [True, True, False]), flush=flush)
    return t_f, t_d, t_w, t_lf, t_lb, flops


def case_conv():
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 256
    torch.backends.cudnn.benchmark = True
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    tot = [0.0] * 5
    print(f"ResNet-50 convolutions, batch {n}, bf16 channels-last; times in us (own kernels: forward incl. BatchNorm "
          "statistics of two view segments | data grad | weight grad; library: forward | data + weight grad)")
    for cin, cout, k, stride, side, count in R50_CONV:
        t_f, t_d, t_w, t_lf, t_lb, flops = _conv_one(cin, cout, k, stride, side, n, flush)
        for i, t in enumerate((t_f, t_d, t_w, t_lf, t_lb)):
            tot[i] += t * count
        print(f"{cin:5d}->{cout:5d} k{k} s{stride} @{side:3d} x{count}: own {t_f:7.1f} {t_d:7.1f} {t_w:7.1f} "
              f"({flops / t_f / 1e6:6.0f} {flops / t_d / 1e6:6.0f} {flops / t_w / 1e6:6.0f} TFLOP/s) | library {t_lf:7.1f} "
              f"{t_lb:7.1f}", flush=True)
    print(f"sum over the network: own fwd {tot[0] / 1e3:.2f} ms, dgrad {tot[1] / 1e3:.2f} ms, wgrad {tot[2] / 1e3:.2f} ms; "
          f"library fwd {tot[3] / 1e3:.2f} ms, bwd {tot[4] / 1e3:.2f} ms")


def case_conv1():
    cin, cout, k, stride, side = (int(v) for v in sys.argv[2:7])
    n = int(sys.argv[7]) if len(sys.argv) > 7 else 256
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    t_f, t_d, t_w, t_lf, t_lb, flops = _conv_one(cin, cout, k, stride, side, n, flush)
    print(f"{cin}->{cout} k{k} s{stride} @{side} batch {n}: own fwd {t_f:.1f} us ({flops / t_f / 1e6:.0f} TFLOP/s), dgrad "
          f"{t_d:.1f} us ({flops / t_d / 1e6:.0f}), wgrad {t_w:.1f} us ({flops / t_w / 1e6:.0f}); library fwd {t_lf:.1f} us, "
          f"bwd {t_lb:.1f} us")


def case_dp():
    """Fused data-parallel LARS over peer memory, launched by torchrun on R GPUs: device time of the reduce-scatter +
    norms kernel and of the update + all-gather kernel on a ResNet-50-sized flat buffer (max over ranks), with the bytes
    each moves over NVLink.  ``dp [N_PARAMS_M]``."""
    import os
    import torch.distributed as dist
    from torch import nn
    from tspipe_b200.comm import peer
    from tspipe_b200.comm.signals import SignalPad
    from tspipe_b200.optim import LARS
    from tspipe_b200.runtime.state import FlatParams
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    n_m = float(sys.argv[2]) if len(sys.argv) > 2 else 25.6
    torch.manual_seed(0)
    n_tensors = 160
    each = int(n_m * 1e6 / n_tensors) // 64 * 64
    params = [nn.Parameter(torch.randn(each, device=dev) * 0.05) for _ in range(n_tensors)]
    flat = FlatParams(params, dev, with_grad=True, pad_to=world)
    opt = LARS(params, lr=0.1, weight_decay=1e-6, momentum=0.9)
    opt.bind_flat(flat, use_kernel=True)
    ranks = list(range(world))
    grads = peer.exchange(flat.grad, dist.group.WORLD, ranks)
    datas = peer.exchange(flat.data, dist.group.WORLD, ranks)
    opt.enable_dp(dist.group.WORLD, grads, datas, rank)
    pad = SignalPad(dist.group.WORLD, ranks, rank, dev, limit_ms=20000)
    table = torch.zeros(world * 2 * n_tensors, dtype=torch.float32, device=dev)
    opt.enable_signals(pad, peer.exchange(table, dist.group.WORLD, ranks))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    t_red, t_step = [], []
    for it in range(13):
        flat.grad.normal_()
        flush.zero_()
        dist.barrier()
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        opt.dp_reduce()
        e[1].record()
        opt.step()
        e[2].record()
        torch.cuda.synchronize()
        if it >= 3:
            t_red.append(e[0].elapsed_time(e[1]) * 1e3)
            t_step.append(e[1].elapsed_time(e[2]) * 1e3)
    pad.check()
    t = torch.tensor([sorted(t_red)[len(t_red) // 2], sorted(t_step)[len(t_step) // 2]], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        total = flat.total * 4
        link = total / world * (world - 1)                # bytes one GPU pulls in (reduce) or pushes out (gather)
        print(f"dp LARS over {world} GPUs, {flat.total / 1e6:.1f} M fp32 parameters: reduce-scatter + norms "
              f"{float(t[0]):.1f} us, update + all-gather {float(t[1]):.1f} us (median of 10, max over ranks, includes "
              f"the signal waits); NVLink bytes per GPU and kernel {link / 1e6:.1f} MB = {link / 770e9 * 1e6:.1f} us at "
              f"770 GB/s; local HBM bytes of the shard {(total / world) * 5 / 1e6:.1f} MB")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    {"bn": case_bn, "bn_r50": case_bn_r50, "stem": case_stem, "lars": case_lars, "ema": case_ema, "kd": case_kd, "ln": case_ln, "gemm": case_gemm,
     "infonce": case_infonce, "attn": case_attn, "conv": case_conv, "conv1": case_conv1, "dp": case_dp}[sys.argv[1]]()
