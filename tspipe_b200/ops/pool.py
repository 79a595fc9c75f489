"""Channels-last 3x3 / stride-2 / pad-1 max pooling and global average pooling (``csrc/pool.cu``) with library
fallbacks."""
from __future__ import annotations

import ctypes as _c

import torch
import torch.nn.functional as F
from torch import nn

from . import fused as _f


class _MaxPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, c, h, w = x.shape
        ho, wo = (h + 1) // 2, (w + 1) // 2
        y = torch.empty((n, c, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        need_idx = x.requires_grad
        idx = torch.empty((n, ho, wo, c), dtype=torch.uint8, device=x.device) if need_idx else None
        L = _f.lib()
        L.tsp_maxpool3x3s2_fwd.restype = _c.c_int
        with _f.on_device(x.device):
            _f._check(L.tsp_maxpool3x3s2_fwd(_f._ptr(x), _f._ptr(y), _f._ptr(idx), _c.c_int(n), _c.c_int(h), _c.c_int(w),
                                             _c.c_int(c), _c.c_int(_f._dt(x)), _f._stream()), "tsp_maxpool3x3s2_fwd")
        _f._count()
        if need_idx:
            ctx.save_for_backward(idx)
        ctx.shape = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        n, c, h, w = ctx.shape
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty((n, c, h, w), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        L = _f.lib()
        L.tsp_maxpool3x3s2_bwd.restype = _c.c_int
        with _f.on_device(dy.device):
            _f._check(L.tsp_maxpool3x3s2_bwd(_f._ptr(dy), _f._ptr(idx), _f._ptr(dx), _c.c_int(n), _c.c_int(h), _c.c_int(w),
                                             _c.c_int(c), _c.c_int(_f._dt(dy)), _f._stream()), "tsp_maxpool3x3s2_bwd")
        _f._count()
        return dx


class MaxPool3x3s2(nn.MaxPool2d):
    """``nn.MaxPool2d(3, stride=2, padding=1)`` that uses the channels-last kernel when it applies."""

    def __init__(self):
        super().__init__(3, stride=2, padding=1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        from . import bn as _bn
        if (x.is_cuda and _bn._ENABLED and x.dim() == 4 and x.shape[1] % 8 == 0
                and x.dtype in (torch.float32, torch.bfloat16) and x.shape[2] > 1
                and x.stride() == (x.shape[2] * x.shape[3] * x.shape[1], 1, x.shape[3] * x.shape[1], x.shape[1])):
            return _MaxPool.apply(x)
        return F.max_pool2d(x, 3, 2, 1)


class _GlobalAvgPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, c, h, w = x.shape
        y = torch.empty((n, c, 1, 1), dtype=x.dtype, device=x.device)
        L = _f.lib()
        L.tsp_avgpool_fwd.restype = _c.c_int
        with _f.on_device(x.device):
            _f._check(L.tsp_avgpool_fwd(_f._ptr(x), _f._ptr(y), _c.c_int(n), _c.c_int(h * w), _c.c_int(c),
                                        _c.c_int(_f._dt(x)), _f._stream()), "tsp_avgpool_fwd")
        _f._count()
        ctx.shape = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        n, c, h, w = ctx.shape
        dy = dy.reshape(n, c).contiguous()
        dx = torch.empty((n, c, h, w), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        L = _f.lib()
        L.tsp_avgpool_bwd.restype = _c.c_int
        with _f.on_device(dy.device):
            _f._check(L.tsp_avgpool_bwd(_f._ptr(dy), _f._ptr(dx), _c.c_int(n), _c.c_int(h * w), _c.c_int(c),
                                        _c.c_int(_f._dt(dy)), _f._stream()), "tsp_avgpool_bwd")
        _f._count()
        return dx


class GlobalAvgPool(nn.AdaptiveAvgPool2d):
    """``nn.AdaptiveAvgPool2d(1)`` that uses the channels-last kernel when it applies (the pooling in front of the
    ResNet heads, `benchmarks/byol/models/resnet_base_network.py` via torchvision's ``avgpool`` in the reference)."""

    def __init__(self):
        super().__init__(1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        from . import bn as _bn
        if (x.is_cuda and _bn._ENABLED and x.dim() == 4 and x.shape[1] % 8 == 0
                and x.dtype in (torch.float32, torch.bfloat16) and x.shape[2] * x.shape[3] > 1
                and x.stride() == (x.shape[2] * x.shape[3] * x.shape[1], 1, x.shape[3] * x.shape[1], x.shape[1])):
            return _GlobalAvgPool.apply(x)
        return F.adaptive_avg_pool2d(x, 1)
