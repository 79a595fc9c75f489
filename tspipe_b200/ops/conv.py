"""Convolutions on the hand-written tcgen05 kernels.

* :func:`conv2d` - 1x1 and 3x3 convolutions (stride 1 or 2, padding (k-1)/2, channel counts multiples of 64) of
  channels-last bf16 activations: forward, data gradient and weight gradient are implicit GEMMs on tcgen05 / TMEM with
  TMA-fetched pixel boxes (``csrc/conv_igemm_tcgen05.cu``); the forward can hand the following BatchNorm its
  per-channel statistics from the epilogue, one set per stacked view.
* :func:`stem_conv` - the ResNet stem (7 x 7, stride 2, 3 -> 64 channels; ``csrc/conv_stem_tcgen05.cu``), also with
  BatchNorm statistics in the epilogue.
* :func:`conv_bn_act` - ``relu(bn(conv(x)) + residual)`` built from the two and :func:`tspipe_b200.ops.bn.bn_act`.

Reference call sites: the convolutions of the torchvision ResNet that
`benchmarks/byol/models/resnet_base_network.py:60-77` flattens (library convolutions there).
"""
from __future__ import annotations

import ctypes as _c
import os
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
        with _f.on_device(x.device):
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
# 1x1 / 3x3 convolutions: implicit GEMM on tcgen05 (csrc/conv_igemm_tcgen05.cu)
# -------------------------------------------------------------------------------------------------
# eligible convolutions run on the tcgen05 implicit-GEMM kernels (set_igemm(False) or TSPIPE_CONV=library: library)
_IGEMM = os.environ.get("TSPIPE_CONV", "igemm") != "library"
_W16 = {}            # id(weight) -> (weight, version, bf16 [Cout, k, k, Cin] copy); dropped at every optimizer step


def set_igemm(flag: bool) -> None:
    """Route eligible convolutions through the tcgen05 implicit-GEMM kernels (default) or the library."""
    global _IGEMM
    _IGEMM = bool(flag)


def clear_weight_cache() -> None:
    _W16.clear()


def _w16(weight: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a convolution weight laid out ``[Cout][kh][kw][Cin]`` (no copy beyond the cast when the
    parameter is stored channels-last, which is how the runtime keeps 4-D parameters)."""
    if _f.IN_CAPTURE:                   # inside a CUDA graph the cast is part of the graph
        w = weight.detach().to(torch.bfloat16).permute(0, 2, 3, 1)
        return w if w.is_contiguous() else w.contiguous()
    hit = _W16.get(id(weight))
    if hit is not None and hit[0] is weight and hit[1] == weight._version and hit[2].device == weight.device:
        return hit[2]
    w = weight.detach().to(torch.bfloat16).permute(0, 2, 3, 1)
    if not w.is_contiguous():
        w = w.contiguous()
    _W16[id(weight)] = (weight, weight._version, w)
    return w


def _nhwc(x: torch.Tensor) -> bool:
    n, c, h, w = x.shape
    return x.stride() == (h * w * c, 1, w * c, c) or (h * w == 1 and x.is_contiguous())


def igemm_eligible(m: nn.Module, x: torch.Tensor) -> bool:
    """Conv2d with a square 1x1 or 3x3 kernel, stride 1 or 2, padding (k-1)/2, no bias / groups / dilation, channel
    counts multiples of 64, on a channels-last bf16 CUDA activation (even height and width for stride 2)."""
    if not (isinstance(m, nn.Conv2d) and m.groups == 1 and m.bias is None and m.dilation == (1, 1)
            and m.padding_mode == "zeros"):
        return False
    k, s = m.kernel_size[0], m.stride[0]
    if m.kernel_size != (k, k) or m.stride != (s, s) or k not in (1, 3) or s not in (1, 2) \
            or m.padding != ((k - 1) // 2, (k - 1) // 2):
        return False
    if m.in_channels % 64 or m.out_channels % 64:
        return False
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16):
        return False
    n, c, h, w = x.shape
    if s == 2 and (h % 2 or w % 2):
        return False
    return _nhwc(x) and x.data_ptr() % 16 == 0


def _lib():
    L = _f.lib()
    if not hasattr(L, "_conv_ready"):
        for name in ("tsp_conv_fprop", "tsp_conv_dgrad", "tsp_conv_wgrad"):
            getattr(L, name).restype = _c.c_int
        L._conv_ready = True
    return L


def _geom(x: torch.Tensor, weight: torch.Tensor, stride: int):
    n, cin, h, w = x.shape
    cout, k = weight.shape[0], weight.shape[2]
    pad = (k - 1) // 2
    return n, h, w, cin, cout, k, (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1


def _stats_ok(n: int, ho: int, wo: int, k: int, stride: int, segs: int) -> bool:
    if n % segs:
        return False
    if k == 1 and stride == 1:
        return (n // segs * ho * wo) % 128 == 0
    if ho * wo <= 64:                          # several images per pixel box: a box must not straddle two views
        per_box = 128 // (ho * wo)
        tiles = -(-n // per_box)
        return (n // segs) % (-(-n // tiles)) == 0
    return True


class _Conv2d(torch.autograd.Function):
    """``conv2d`` forward / backward on the implicit-GEMM kernels.  Returns ``(y, sums)``; ``sums`` (not
    differentiable) holds ``[segs][sum | sum of squares]`` per output channel when requested."""

    @staticmethod
    def forward(ctx, x, weight, stride, want_sums, segs):
        n, h, w, cin, cout, k, ho, wo = _geom(x, weight, stride)
        w16 = _w16(weight)
        y = torch.empty((n, cout, ho, wo), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
        sums = torch.zeros(segs * 2 * cout, dtype=torch.float32, device=x.device) if want_sums else None
        with _f.on_device(x.device):
            code = _lib().tsp_conv_fprop(_f._ptr(x), _f._ptr(w16), _f._ptr(y), _f._ptr(sums), _c.c_int(segs), _c.c_int(n),
                                         _c.c_int(h), _c.c_int(w), _c.c_int(cin), _c.c_int(cout), _c.c_int(k),
                                         _c.c_int(stride), _f._ptr(_gemm._status_word(x.device)), _f._stream())
        _f._check(code, "tsp_conv_fprop")
        _f._count()
        ctx.save_for_backward(x, weight)
        ctx.stride = stride
        if sums is None:
            sums = torch.empty(0, device=x.device)
        ctx.mark_non_differentiable(sums)
        return y, sums

    @staticmethod
    def backward(ctx, dy, _dsums):
        x, weight = ctx.saved_tensors
        stride = ctx.stride
        n, h, w, cin, cout, k, ho, wo = _geom(x, weight, stride)
        if dy.dtype != torch.bfloat16 or not _nhwc(dy):
            dy = dy.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        L = _lib()
        status = _f._ptr(_gemm._status_word(x.device))
        dx = dw = None
        with _f.on_device(x.device):
            st = _f._stream()
            if ctx.needs_input_grad[0]:
                dx = torch.empty_like(x)
                code = L.tsp_conv_dgrad(_f._ptr(dy), _f._ptr(_w16(weight)), _f._ptr(dx), _c.c_int(n), _c.c_int(h),
                                        _c.c_int(w), _c.c_int(cin), _c.c_int(cout), _c.c_int(k), _c.c_int(stride),
                                        status, st)
                _f._check(code, "tsp_conv_dgrad")
                _f._count(4 if stride == 2 and k == 3 else 1)
            if ctx.needs_input_grad[1]:
                # The kernel ADDS into its output.  When the parameter's gradient already lives in an fp32 buffer of
                # the kernel's layout ([Cout][k][k][Cin], i.e. channels-last, as in the runtime's flat gradient
                # buffer) the sum goes straight there and autograd gets nothing more to accumulate.
                g = weight.grad if weight.is_leaf else None
                if (_ACCUMULATE_IN_PLACE and g is not None and g.dtype == torch.float32 and g.shape == weight.shape
                        and g.permute(0, 2, 3, 1).is_contiguous()):
                    target = g
                else:
                    target = torch.zeros((cout, k, k, cin), dtype=torch.float32, device=x.device)
                    dw = target.permute(0, 3, 1, 2)
                code = L.tsp_conv_wgrad(_f._ptr(x), _f._ptr(dy), _f._ptr(target), _c.c_int(n), _c.c_int(h), _c.c_int(w),
                                        _c.c_int(cin), _c.c_int(cout), _c.c_int(k), _c.c_int(stride), status, st)
                _f._check(code, "tsp_conv_wgrad")
                _f._count()
                if dw is not None and weight.dtype != torch.float32:
                    dw = dw.to(weight.dtype)
        return dx, dw, None, None, None


_ACCUMULATE_IN_PLACE = True


def set_accumulate_in_place(flag: bool) -> None:
    """Let the weight-gradient kernel add straight into an existing fp32 ``weight.grad`` of matching layout (default)
    instead of handing autograd a fresh tensor to accumulate."""
    global _ACCUMULATE_IN_PLACE
    _ACCUMULATE_IN_PLACE = bool(flag)


def conv2d(x: torch.Tensor, weight: torch.Tensor, stride: int = 1, want_sums: bool = False, segments: int = 1
           ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``(y, sums)``: ``y = conv2d(x, weight, stride, padding (k-1)/2)`` in channels-last bf16; ``sums`` =
    ``[segments][sum | sum of squares]`` per output channel over each group of ``N / segments`` consecutive images
    (fp32) when ``want_sums`` and the tiling allows it, else None."""
    n, h, w, cin, cout, k, ho, wo = _geom(x, weight, stride)
    want = bool(want_sums) and _stats_ok(n, ho, wo, k, stride, segments)
    y, sums = _Conv2d.apply(x, weight, stride, want, segments)
    return y, (sums if want else None)


def conv_bn_act(conv: nn.Module, bn: nn.Module, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                relu: bool = False) -> torch.Tensor:
    """``relu(bn(conv(x)) + residual)``.  An eligible convolution runs on the tcgen05 implicit-GEMM kernel; in front
    of a training-mode BatchNorm its epilogue already produces the BatchNorm's statistics (one pass over the
    activation less).  Everything else is the library convolution followed by :func:`tspipe_b200.ops.bn.bn_act`."""
    from . import bn as _bn
    if _IGEMM and torch.is_autocast_enabled() and igemm_eligible(conv, x):
        want = bool(bn.training)
        segs = _bn.current_segments() if want else 1
        y, sums = conv2d(x, conv.weight, conv.stride[0], want_sums=want, segments=segs)
        return _bn.bn_act(bn, y, residual, relu, sums=sums if (sums is not None and _bn.applicable(bn, y)) else None)
    return _bn.bn_act(bn, conv(x), residual, relu)


def conv(m: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """``m(x)`` for a Conv2d, on the implicit-GEMM kernel when eligible."""
    if _IGEMM and torch.is_autocast_enabled() and igemm_eligible(m, x):
        return conv2d(x, m.weight, m.stride[0])[0]
    return m(x)
