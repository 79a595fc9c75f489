"""Convolutions with their own tcgen05 kernels, each with the following BatchNorm's statistics computed in the
epilogue: the ResNet stem (7 x 7, stride 2, 3 -> 64 channels; ``csrc/conv_stem_tcgen05.cu``) and 1 x 1 stride-1
convolutions of channels-last activations, which are plain GEMMs (``csrc/gemm_tcgen05_2cta.cu``, statistics variant).

Reference call site: ``conv1`` of the torchvision ResNet that `benchmarks/byol/models/resnet_base_network.py`
wraps (a library convolution there).  The weight gradient stays a library call
(``aten::convolution_backward``); the layer's input needs no gradient.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch
from torch import nn

from . import fused as _f
from . import gemm as _gemm

K_REAL = 147
K_PAD = 192


def is_stem_conv(m: nn.Module) -> bool:
    return (isinstance(m, nn.Conv2d) and m.in_channels == 3 and m.out_channels == 64 and m.kernel_size == (7, 7)
            and m.stride == (2, 2) and m.padding == (3, 3) and m.dilation == (1, 1) and m.groups == 1
            and m.bias is None and m.padding_mode == "zeros")


def eligible(x: torch.Tensor) -> bool:
    """Channels-last bf16 CUDA input [N, 3, H, W] with H even and W a multiple of 8 in [8, 224]."""
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16):
        return False
    n, c, h, w = x.shape
    if c != 3 or h % 2 or w % 8 or not (8 <= w <= 224) or h < 8:
        return False
    return x.stride() == (h * w * 3, 1, w * 3, 3) and x.data_ptr() % 16 == 0


def weight_matrix(weight: torch.Tensor) -> torch.Tensor:
    """``[64, 3, 7, 7]`` -> bf16 ``[64, 192]`` with ``k = kh * 21 + kw * 3 + c`` and zeros from k = 147."""
    wm = torch.zeros(64, K_PAD, dtype=torch.bfloat16, device=weight.device)
    wm[:, :K_REAL] = weight.detach().permute(0, 2, 3, 1).reshape(64, K_REAL)
    return wm


class _StemConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, want_sums, segs):
        n, _, h, w = x.shape
        y = torch.empty((n, 64, h // 2, w // 2), dtype=torch.bfloat16, device=x.device,
                        memory_format=torch.channels_last)
        sums = torch.zeros(segs * 128, dtype=torch.float32, device=x.device) if want_sums else None
        wm = weight_matrix(weight)
        L = _f.lib()
        L.tsp_conv_stem_fwd.restype = _c.c_int
        with torch.cuda.device(x.device):
            code = L.tsp_conv_stem_fwd(_f._ptr(x), _f._ptr(wm), _f._ptr(y), _f._ptr(sums), _c.c_int(n), _c.c_int(h),
                                       _c.c_int(w), _c.c_int(segs), _f._ptr(_gemm._status_word(x.device)), _f._stream())
        _f._check(code, "tsp_conv_stem_fwd")
        _f._count()
        ctx.save_for_backward(x, weight)
        if sums is None:
            sums = torch.empty(0, device=x.device)
        ctx.mark_non_differentiable(sums)
        return y, sums

    @staticmethod
    def backward(ctx, dy, _dsums):
        x, weight = ctx.saved_tensors
        dx = dw = None
        need_dx = ctx.needs_input_grad[0]
        gi, gw, _ = torch.ops.aten.convolution_backward(
            dy.contiguous(memory_format=torch.channels_last), x, weight.to(torch.bfloat16), None, [2, 2], [3, 3],
            [1, 1], False, [0, 0], 1, [need_dx, ctx.needs_input_grad[1], False])
        if need_dx:
            dx = gi
        if ctx.needs_input_grad[1]:
            dw = gw.to(weight.dtype)
        return dx, dw, None, None


def stem_conv(x: torch.Tensor, weight: torch.Tensor, want_sums: bool = True, segments: int = 1
              ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``(y, sums)``: y = conv2d(x, weight, stride 2, padding 3) in channels-last bf16; ``sums`` = per-channel
    [sum | sum of squares] of y over all pixels (fp32, ``[segments][128]`` flattened: one set per group of
    ``N / segments`` consecutive images) or None."""
    if x.shape[0] % segments != 0:
        segments = 1
    y, sums = _StemConv.apply(x, weight, want_sums, segments)
    return y, (sums if want_sums else None)


# -------------------------------------------------------------------------------------------------
# 1 x 1 convolution = GEMM over the [N*H*W, Cin] view of a channels-last activation
# -------------------------------------------------------------------------------------------------
_CONV1X1 = False
_PAIR = False        # CTA-pair kernel instead of one CTA per tile (the latter is faster on tall, narrow products)
_MIN_COUT = 256      # narrower outputs: the library convolution plus a statistics pass is as fast or faster
_W16 = {}        # id(weight) -> bf16 [Cout, Cin] copy; dropped at every optimizer step (clear_weight_cache)


def set_conv1x1(flag: bool) -> None:
    """Route eligible 1 x 1 convolutions that feed a training-mode BatchNorm through the tcgen05 GEMM."""
    global _CONV1X1
    _CONV1X1 = bool(flag)


def clear_weight_cache() -> None:
    _W16.clear()


def _w16(weight: torch.Tensor) -> torch.Tensor:
    w = _W16.get(id(weight))
    if w is None or w.device != weight.device:
        w = weight.detach().reshape(weight.shape[0], weight.shape[1]).to(torch.bfloat16).contiguous()
        _W16[id(weight)] = w
    return w


def conv1x1_eligible(m: nn.Module, x: torch.Tensor, segments: int = 1) -> bool:
    if not (isinstance(m, nn.Conv2d) and m.kernel_size == (1, 1) and m.stride == (1, 1) and m.padding == (0, 0)
            and m.groups == 1 and m.bias is None):
        return False
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16):
        return False
    n, c, h, w = x.shape
    rows = n * h * w
    if c % 8 or m.out_channels % 8 or c < 64 or m.out_channels < _MIN_COUT or rows % segments \
            or (rows // segments) % 128:
        return False
    return x.stride() == (h * w * c, 1, w * c, c) and x.data_ptr() % 16 == 0


class _Conv1x1(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, segs):
        n, cin, h, w = x.shape
        cout = weight.shape[0]
        rows = n * h * w
        w16 = _w16(weight)
        y = torch.empty((n, cout, h, w), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
        sums = torch.zeros(segs * 2 * cout, dtype=torch.float32, device=x.device)
        L = _f.lib()
        fn = L.tsp_gemm_bf16_tn_2cta_stats if _PAIR else L.tsp_gemm_bf16_tn_stats
        fn.restype = _c.c_int
        with torch.cuda.device(x.device):
            code = fn(_f._ptr(x), _f._ptr(w16), _f._ptr(y), _c.c_int(rows), _c.c_int(cout),
                                                 _c.c_int(cin), _c.c_int(cin), _c.c_int(cin), _c.c_int(cout),
                                                 _f._ptr(sums), _c.c_int(segs), _f._ptr(_gemm._status_word(x.device)),
                                                 _f._stream())
        _f._check(code, "tsp_gemm_bf16_tn_stats")
        _f._count()
        ctx.save_for_backward(x, weight)
        ctx.mark_non_differentiable(sums)
        return y, sums

    @staticmethod
    def backward(ctx, dy, _dsums):
        x, weight = ctx.saved_tensors
        w4 = _w16(weight).view(weight.shape[0], weight.shape[1], 1, 1)
        gi, gw, _ = torch.ops.aten.convolution_backward(
            dy.contiguous(memory_format=torch.channels_last), x, w4, None, [1, 1], [0, 0], [1, 1], False, [0, 0], 1,
            [ctx.needs_input_grad[0], ctx.needs_input_grad[1], False])
        return gi, (gw.to(weight.dtype) if gw is not None else None), None


def conv1x1(x: torch.Tensor, weight: torch.Tensor, segments: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(y, sums)`` for a 1 x 1 stride-1 convolution of a channels-last bf16 activation: ``y`` bf16 channels-last,
    ``sums`` = ``[segments][sum | sum of squares]`` per output channel (fp32) over each group of rows."""
    return _Conv1x1.apply(x, weight, segments)


def conv_bn_act(conv: nn.Module, bn: nn.Module, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                relu: bool = False) -> torch.Tensor:
    """``relu(bn(conv(x)) + residual)``.  A 1 x 1 stride-1 convolution in front of a training-mode BatchNorm runs on
    the tcgen05 GEMM whose epilogue already produces the BatchNorm's statistics (one pass over the activation
    less); everything else is the library convolution followed by :func:`tspipe_b200.ops.bn.bn_act`."""
    from . import bn as _bn
    if _CONV1X1 and bn.training and torch.is_autocast_enabled():
        segs = _bn.current_segments()
        if conv1x1_eligible(conv, x, segs):
            y, sums = conv1x1(x, conv.weight, segs)
            return _bn.bn_act(bn, y, residual, relu, sums=sums if _bn.applicable(bn, y) else None)
    return _bn.bn_act(bn, conv(x), residual, relu)
