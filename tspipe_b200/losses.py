"""Loss functions with the reference's callback signatures, picklable (module level).

``soft_target_kd``: ``CE + lambda_kd * T^2 * KL(softmax(t/T) || log_softmax(s/T))`` (batchmean), the
reference's objective (`benchmarks/soft_target/kd_losses/st.py:18-23`,
`benchmarks/soft_target/train_kd.py:439-453`, ``--lambda_kd`` default 1.0); a caller that passes ``alpha``
instead gets the convex mix ``(1 - alpha) * CE + alpha * T^2 * KL``.  ``logits_kd``: the same with the MSE
between the logits in place of the KL term (`benchmarks/soft_target/kd_losses/logits.py:17-20`).
``byol_loss``: 2 - 2 cos, symmetric, batch mean (`benchmarks/byol/trainer.py:51-55,192-196`).
``moco_loss``: InfoNCE with temperature, x 2T, symmetric (`benchmarks/moco-v3/main.py:147-162`).
``ema_update``: ``m*t + (1-m)*s`` (`benchmarks/byol/trainer.py:198-212`); it carries the
``is_ema`` marker that lets the runtime replace it by the fused in-place kernel.

On CUDA with ``runtime.fused`` these dispatch to the sm_100a kernels in
:mod:`tspipe_b200.ops.fused`; otherwise they are the plain PyTorch expressions.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F


def _fused_ok(*ts: torch.Tensor) -> bool:
    if not all(t.is_cuda for t in ts):
        return False
    from .ops import fused
    return fused.available()


def kd_weights(extra_args) -> tuple:
    """``(w_ce, w_kd)``: ``lambda_kd`` gives the reference's ``CE + lambda_kd * KD`` (default ``lambda_kd = 1``,
    `benchmarks/soft_target/train_kd.py:62,448-453`); ``alpha`` gives ``(1 - alpha) * CE + alpha * KD``."""
    if getattr(extra_args, "lambda_kd", None) is not None:
        return 1.0, float(extra_args.lambda_kd)
    if getattr(extra_args, "alpha", None) is not None:
        a = float(extra_args.alpha)
        return 1.0 - a, a
    return 1.0, 1.0


def soft_target_kd(student_out, teacher_out, labels, args=None, extra_args=None, epoch: int = 0):
    T = float(getattr(extra_args, "T", 4.0))
    w_ce, w_kd = kd_weights(extra_args)
    if _fused_ok(student_out, teacher_out) and not getattr(extra_args, "no_fused", False):
        from .ops import fused
        return fused.kd_soft_target_loss(student_out, teacher_out, labels, T, w_ce, w_kd)
    ce = F.cross_entropy(student_out.float(), labels)
    kd = F.kl_div(F.log_softmax(student_out.float() / T, dim=1), F.softmax(teacher_out.float() / T, dim=1),
                  reduction="batchmean") * T * T
    return w_ce * ce + w_kd * kd


def logits_kd(student_out, teacher_out, labels, args=None, extra_args=None, epoch: int = 0):
    """"Do deep nets really need to be deep": MSE between student and teacher logits plus CE
    (`benchmarks/soft_target/kd_losses/logits.py:17-20`, `train_kd.py:448-453`)."""
    w_ce, w_kd = kd_weights(extra_args)
    t = teacher_out if isinstance(teacher_out, torch.Tensor) else None
    if t is None:
        raise TypeError("logits_kd needs the teacher logits as a tensor")
    return w_ce * F.cross_entropy(student_out.float(), labels) + w_kd * F.mse_loss(student_out.float(), t.float())


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


def _info_nce(q: torch.Tensor, k: torch.Tensor, T: float, label_offset: int = 0) -> torch.Tensor:
    q = F.normalize(q.float(), dim=1)
    k = F.normalize(k.float(), dim=1)
    logits = q @ k.t() / T
    labels = torch.arange(logits.shape[0], device=logits.device) + label_offset
    return F.cross_entropy(logits, labels) * (2 * T)


def moco_loss(online_view_1, online_view_2, target_view_1, target_view_2, args=None, extra_args=None):
    """Symmetric InfoNCE (`benchmarks/moco-v3/main.py:147-162`).  With data-parallel pipeline replicas the keys of
    all replicas are gathered first and the positives sit at ``arange(n) + n * replica``
    (`benchmarks/moco-v3/moco/builder.py:73-85`)."""
    from .parallel.keys import gather_keys
    T = float(getattr(extra_args, "moco_t", 0.2))
    if _fused_ok(online_view_1, target_view_2) and not getattr(extra_args, "no_fused", False):
        from .ops import gemm
        l1 = gemm.info_nce_replicas(online_view_1, target_view_2, T)
        if l1 is not None:
            return l1 + gemm.info_nce_replicas(online_view_2, target_view_1, T)
    k2, off = gather_keys(target_view_2)
    k1, _ = gather_keys(target_view_1)
    if _fused_ok(online_view_1, target_view_2) and not getattr(extra_args, "no_fused", False):
        from .ops import gemm
        return gemm.info_nce(online_view_1, target_view_2, T, k2, off) + \
            gemm.info_nce(online_view_2, target_view_1, T, k1, off)
    return _info_nce(online_view_1, k2, T, off) + _info_nce(online_view_2, k1, T, off)


def distil_loss(student_out, teacher_out, labels, args=None, extra_args=None, epoch: int = 0):
    """DistilBERT objective (`benchmarks/distilbert/distiller.py:711-772`):
    ``alpha_ce * T^2 * KL(softmax(t/T) || softmax(s/T))`` over the tokens selected by the attention mask
    (batch-mean over selected tokens) ``+ alpha_mlm * CE(s, lm_labels)`` (mean over labelled tokens,
    ``-100`` ignored) ``+ alpha_cos * (1 - cos(h_s, h_t))`` over the selected tokens.

    ``student_out`` / ``teacher_out`` are ``(logits [B, L, V], last_hidden [B, L, H])``; ``labels`` is
    ``(lm_labels [B, L], attention_mask [B, L])`` optionally followed by the two token counts as Python
    ints (saves a device synchronisation)."""
    s_logits, s_hidden = student_out
    t_logits, t_hidden = teacher_out
    lm_labels, attn = labels[0], labels[1]
    T = float(getattr(extra_args, "temperature", 2.0))
    a_ce = float(getattr(extra_args, "alpha_ce", 5.0))
    a_mlm = float(getattr(extra_args, "alpha_mlm", 2.0))
    a_cos = float(getattr(extra_args, "alpha_cos", 1.0))
    sel = attn.to(torch.bool)
    n_sel = int(labels[3]) if len(labels) > 3 else int(sel.sum())
    n_lab = int(labels[2]) if len(labels) > 2 else int((lm_labels >= 0).sum())
    n_sel, n_lab = max(n_sel, 1), max(n_lab, 1)
    if _fused_ok(s_logits, t_logits) and not getattr(extra_args, "no_fused", False):
        from .ops import fused
        loss = fused.kd_ce_loss(s_logits, t_logits, lm_labels, T, a_mlm / n_lab, a_ce / n_sel, row_mask=sel)
        if a_cos > 0:
            loss = loss + fused.cosine_embedding_loss(s_hidden, t_hidden, a_cos / n_sel, row_mask=sel)
        return loss
    v = s_logits.shape[-1]
    s_sel = s_logits.float()[sel]
    t_sel = t_logits.float()[sel]
    loss = a_ce * F.kl_div(F.log_softmax(s_sel / T, dim=-1), F.softmax(t_sel / T, dim=-1),
                           reduction="batchmean") * T * T
    loss = loss + a_mlm * F.cross_entropy(s_logits.float().view(-1, v), lm_labels.view(-1), ignore_index=-100)
    if a_cos > 0:
        hs, ht = s_hidden.float()[sel], t_hidden.float()[sel]
        loss = loss + a_cos * F.cosine_embedding_loss(hs, ht, torch.ones(hs.shape[0], device=hs.device))
    return loss


@torch.no_grad()
def _ema_reference(m: float, online_new_param: List[torch.Tensor], target_param: List[torch.Tensor]):
    return [t.detach() * m + s.detach() * (1.0 - m) for s, t in zip(online_new_param, target_param)]


def ema_update(m: float, online_new_param, target_param=None):
    return _ema_reference(m, online_new_param, target_param)


ema_update.is_ema = True
ema_update.reference_fn = _ema_reference
