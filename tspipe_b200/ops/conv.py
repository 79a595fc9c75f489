"""ResNet stem convolution (7 x 7, stride 2, 3 -> 64 channels) on the tcgen05 kernel of
``csrc/conv_stem_tcgen05.cu``, with the following BatchNorm's statistics computed in its epilogue.

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
