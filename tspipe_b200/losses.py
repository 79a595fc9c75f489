"""Loss functions with the reference's callback signatures, picklable (module level).

``soft_target_kd``: CE + T^2 * KL(softmax(t/T) || log_softmax(s/T)) batchmean
(`benchmarks/soft_target/kd_losses/st.py:18-23`, `benchmarks/soft_target/train_kd.py:439-453`).
``byol_loss``: 2 - 2 cos, symmetric, batch mean (`benchmarks/byol/trainer.py:51-55,192-196`).
``moco_loss``: InfoNCE with temperature, x 2T, symmetric (`benchmarks/moco-v3/main.py:147-162`).
``ema_update``: ``m*t + (1-m)*s`` (`benchmarks/byol/trainer.py:198-212`); it carries the
``is_ema`` marker that lets the runtime replace it by the fused in-place kernel.

On CUDA with ``runtime.fused`` these dispatch to the sm_100a kernels in
:mod:`tspipe_b200.ops.fused`; otherwise they are the plain PyTorch expressions.
"""
from __future__ import annotations

from typing import Any, List, Optional

import torch
import torch.nn.functional as F


def _fused_ok(*ts: torch.Tensor) -> bool:
    if not all(t.is_cuda for t in ts):
        return False
    from .ops import fused
    return fused.available()


def soft_target_kd(student_out, teacher_out, labels, args=None, extra_args=None, epoch: int = 0):
    T = float(getattr(extra_args, "T", 4.0))
    alpha = float(getattr(extra_args, "alpha", getattr(extra_args, "lambda_kd", 0.9)))
    if _fused_ok(student_out, teacher_out) and not getattr(extra_args, "no_fused", False):
        from .ops import fused
        return fused.kd_soft_target_loss(student_out, teacher_out, labels, T, alpha)
    ce = F.cross_entropy(student_out.float(), labels)
    kd = F.kl_div(F.log_softmax(student_out.float() / T, dim=1), F.softmax(teacher_out.float() / T, dim=1),
                  reduction="batchmean") * T * T
    return (1.0 - alpha) * ce + alpha * kd


def regression_loss(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    x = F.normalize(x.float(), dim=1)
    y = F.normalize(y.float(), dim=1)
    return 2 - 2 * (x * y).sum(dim=-1)


def byol_loss(online_view_1, online_view_2, target_view_1, target_view_2, args=None, extra_args=None):
    if _fused_ok(online_view_1, target_view_2) and not getattr(extra_args, "no_fused", False):
        from .ops import fused
        return fused.byol_loss(online_view_1, online_view_2, target_view_1, target_view_2)
    loss = regression_loss(online_view_1, target_view_2) + regression_loss(online_view_2, target_view_1)
    return loss.mean()


def _info_nce(q: torch.Tensor, k: torch.Tensor, T: float) -> torch.Tensor:
    q = F.normalize(q.float(), dim=1)
    k = F.normalize(k.float(), dim=1)
    logits = q @ k.t() / T
    labels = torch.arange(logits.shape[0], device=logits.device)
    return F.cross_entropy(logits, labels) * (2 * T)


def moco_loss(online_view_1, online_view_2, target_view_1, target_view_2, args=None, extra_args=None):
    T = float(getattr(extra_args, "moco_t", 0.2))
    if _fused_ok(online_view_1, target_view_2) and not getattr(extra_args, "no_fused", False):
        from .ops import fused
        return fused.info_nce_loss(online_view_1, target_view_2, T) + fused.info_nce_loss(online_view_2, target_view_1, T)
    return _info_nce(online_view_1, target_view_2, T) + _info_nce(online_view_2, target_view_1, T)


@torch.no_grad()
def _ema_reference(m: float, online_new_param: List[torch.Tensor], target_param: List[torch.Tensor]):
    return [t.detach() * m + s.detach() * (1.0 - m) for s, t in zip(online_new_param, target_param)]


def ema_update(m: float, online_new_param, target_param=None):
    return _ema_reference(m, online_new_param, target_param)


ema_update.is_ema = True
ema_update.reference_fn = _ema_reference
