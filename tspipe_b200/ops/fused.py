"""Python bindings and autograd wrappers of the sm_100a kernels in ``csrc/``.

Every wrapper runs on the current CUDA stream.  ``LAUNCHES`` counts kernel launches issued
through this module (benchmarks report it).  The module raises instead of falling back when the
library cannot be loaded on a CUDA machine.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import build as _build

LAUNCHES = 0
_lib = None
_c = ctypes


def available() -> bool:
    return torch.cuda.is_available()


def lib():
    global _lib
    if _lib is None:
        L = _build.load()
        for name in ("tsp_ema_update", "tsp_lars_step", "tsp_lars_norms", "tsp_lars_apply", "tsp_adamw_step",
                     "tsp_sgd_step", "tsp_byol_loss", "tsp_cosine_loss", "tsp_kd_ce_loss", "tsp_layernorm_fwd",
                     "tsp_layernorm_bwd", "tsp_layernorm_bwd_blocks", "tsp_gelu_fwd", "tsp_gelu_bwd"):
            getattr(L, name).restype = _c.c_int
        _lib = L
    return _lib


def set_sm_reserve(n: int) -> None:
    """Leave ``n`` SMs free of the persistent tcgen05 kernels (convolutions, GEMMs) so that communication kernels
    that become ready while one of them runs - NCCL sends / receives of the stage links, peer reductions on a side
    stream - find an SM at once instead of when the persistent kernel ends."""
    lib().tsp_set_sm_reserve(_c.c_int(int(n)))


def _count(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


def _ptr(t: Optional[torch.Tensor]):
    return _c.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    """Raw handle of the current stream of the current device (the launchers' last argument)."""
    return _c.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


IN_CAPTURE = 0          # > 0 while a stage is being recorded into a CUDA graph


class capturing:
    """While a stage is recorded into a CUDA graph the per-step caches of derived tensors (bf16 weight copies) are
    bypassed: what the graph needs it must compute itself at every replay."""

    def __enter__(self):
        global IN_CAPTURE
        IN_CAPTURE += 1
        return self

    def __exit__(self, *exc):
        global IN_CAPTURE
        IN_CAPTURE -= 1
        return False


class _Current:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_CURRENT = _Current()


def on_device(device):
    """``with on_device(t.device):`` makes the tensor's device current for the launches inside.  Free when it already
    is (every launch of a training step: the executor thread and autograd's device thread both run with their device
    current), so the per-launch cost of the general context manager is only paid when it does something."""
    idx = device.index
    if idx is None or torch._C._cuda_getDevice() == idx:
        return _CURRENT
    return torch.cuda.device(idx)


def _check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}")


# ---------------------------------------------------------------------------------------------
# flat-buffer updates
# ---------------------------------------------------------------------------------------------
@torch.no_grad()
def ema_update_(teacher: torch.Tensor, student: torch.Tensor, momentum: float,
                bf16_shadow: Optional[torch.Tensor] = None) -> None:
    """``teacher = m*teacher + (1-m)*student`` in place (fp32, contiguous).  ``student`` may be a
    view of another GPU's memory mapped into this process."""
    assert teacher.dtype == torch.float32 and student.dtype == torch.float32
    assert teacher.is_contiguous() and student.is_contiguous() and teacher.numel() == student.numel()
    if teacher.numel() == 0:
        return
    with on_device(teacher.device):
        _check(lib().tsp_ema_update(_ptr(teacher), _ptr(student), _c.c_int64(teacher.numel()),
                                    _c.c_float(momentum), _ptr(bf16_shadow), _stream()), "tsp_ema_update")
    _count()


CHUNK = 16384


def build_chunks(offsets: Sequence[int], numels: Sequence[int], device, lo: int = 0, hi: Optional[int] = None
                 ) -> torch.Tensor:
    """Chunk table ``[n_chunks, 3] = (segment, begin, length)`` restricted to flat range ``[lo, hi)``."""
    rows = []
    for s, (off, n) in enumerate(zip(offsets, numels)):
        a, b = max(off, lo), min(off + n, hi if hi is not None else off + n)
        pos = a
        while pos < b:
            ln = min(CHUNK, b - pos)
            rows.append((s, pos, ln))
            pos += ln
    if not rows:
        return torch.zeros((0, 3), dtype=torch.int64, device=device)
    return torch.tensor(rows, dtype=torch.int64, device=device)


@torch.no_grad()
def lars_step_(p, g, mu, chunks, seg_hp, norms, grad_scale=1.0, teacher=None, ema_m=0.0) -> None:
    n_seg = seg_hp.shape[0]
    with on_device(p.device):
        _check(lib().tsp_lars_step(_ptr(p), _ptr(g), _ptr(mu), _ptr(chunks), _c.c_int(chunks.shape[0]), _ptr(seg_hp),
                                   _c.c_float(grad_scale), _ptr(norms), _c.c_int(n_seg), _ptr(teacher),
                                   _c.c_int64(0 if teacher is None else teacher.numel()), _c.c_float(ema_m),
                                   _stream()), "tsp_lars_step")
    _count(3)


@torch.no_grad()
def lars_norms_(p, g, chunks, seg_hp, norms, grad_scale=1.0) -> None:
    with on_device(p.device):
        _check(lib().tsp_lars_norms(_ptr(p), _ptr(g), _ptr(chunks), _c.c_int(chunks.shape[0]), _ptr(seg_hp),
                                    _c.c_float(grad_scale), _ptr(norms), _c.c_int(seg_hp.shape[0]), _stream()),
               "tsp_lars_norms")
    _count(2)


@torch.no_grad()
def lars_apply_(p, g, mu, chunks, seg_hp, norms, grad_scale=1.0, teacher=None, ema_m=0.0) -> None:
    with on_device(p.device):
        _check(lib().tsp_lars_apply(_ptr(p), _ptr(g), _ptr(mu), _ptr(chunks), _c.c_int(chunks.shape[0]), _ptr(seg_hp),
                                    _c.c_float(grad_scale), _ptr(norms), _ptr(teacher),
                                    _c.c_int64(0 if teacher is None else teacher.numel()), _c.c_float(ema_m),
                                    _stream()), "tsp_lars_apply")
    _count()


@torch.no_grad()
def adamw_step_(p, g, m, v, chunks, seg_hp, grad_scale=1.0, teacher=None, ema_m=0.0) -> None:
    with on_device(p.device):
        _check(lib().tsp_adamw_step(_ptr(p), _ptr(g), _ptr(m), _ptr(v), _ptr(chunks), _c.c_int(chunks.shape[0]),
                                    _ptr(seg_hp), _c.c_float(grad_scale), _ptr(teacher),
                                    _c.c_int64(0 if teacher is None else teacher.numel()), _c.c_float(ema_m),
                                    _stream()), "tsp_adamw_step")
    _count()


@torch.no_grad()
def sgd_step_(p, g, buf, chunks, seg_hp, grad_scale=1.0, teacher=None, ema_m=0.0) -> None:
    with on_device(p.device):
        _check(lib().tsp_sgd_step(_ptr(p), _ptr(g), _ptr(buf), _ptr(chunks), _c.c_int(chunks.shape[0]), _ptr(seg_hp),
                                  _c.c_float(grad_scale), _ptr(teacher),
                                  _c.c_int64(0 if teacher is None else teacher.numel()), _c.c_float(ema_m), _stream()),
               "tsp_sgd_step")
    _count()


# ---------------------------------------------------------------------------------------------
# losses: forward computes value AND gradient; backward only scales
# ---------------------------------------------------------------------------------------------
class _ByolPair(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, scale):
        x = x.contiguous()
        y = y.detach().to(x.dtype).contiguous()
        n, d = x.shape
        loss = torch.zeros((), dtype=torch.float32, device=x.device)
        gx = torch.empty_like(x)
        with on_device(x.device):
            _check(lib().tsp_byol_loss(_ptr(x), _ptr(y), _c.c_int(n), _c.c_int(d), _c.c_int(_dt(x)),
                                       _c.c_float(scale), _ptr(loss), _ptr(gx), _stream()), "tsp_byol_loss")
        _count()
        ctx.save_for_backward(gx)
        return loss

    @staticmethod
    def backward(ctx, gout):
        (gx,) = ctx.saved_tensors
        return gx * gout.to(gx.dtype), None, None


def byol_pair_loss(x: torch.Tensor, y: torch.Tensor, scale: float) -> torch.Tensor:
    """``scale * sum_rows (2 - 2 cos(x_r, y_r))``; ``y`` (teacher) gets no gradient and may live in
    peer memory."""
    return _ByolPair.apply(x, y, scale)


def byol_loss(o1, o2, t1, t2) -> torch.Tensor:
    n = o1.shape[0]
    return byol_pair_loss(o1, t2, 1.0 / n) + byol_pair_loss(o2, t1, 1.0 / n)


class _KdCe(torch.autograd.Function):
    @staticmethod
    def forward(ctx, s, t, labels, row_mask, temp, w_ce, w_kd):
        s2 = s.reshape(-1, s.shape[-1]).contiguous()
        if t is None or not isinstance(t, torch.Tensor):
            t2 = t          # None, or a peer-mapped [rows, classes] matrix read in place over NVLink
        else:
            t2 = t.detach().reshape(-1, t.shape[-1]).contiguous()
        n, c = s2.shape
        loss = torch.zeros((), dtype=torch.float32, device=s.device)
        gs = torch.empty_like(s2)
        lab = None if labels is None else labels.reshape(-1).to(torch.int64).contiguous()
        msk = None if row_mask is None else row_mask.reshape(-1).to(torch.uint8).contiguous()
        with on_device(s.device):
            _check(lib().tsp_kd_ce_loss(_ptr(s2), _ptr(t2), _ptr(lab), _ptr(msk), _c.c_int(n), _c.c_int(c),
                                        _c.c_int(_dt(s2)), _c.c_int(0 if t2 is None else _dt(t2)), _c.c_float(temp),
                                        _c.c_float(w_ce), _c.c_float(w_kd), _ptr(loss), _ptr(gs), _stream()),
                   "tsp_kd_ce_loss")
        _count()
        ctx.save_for_backward(gs)
        ctx.shape = s.shape
        return loss

    @staticmethod
    def backward(ctx, gout):
        (gs,) = ctx.saved_tensors
        return (gs * gout.to(gs.dtype)).view(ctx.shape), None, None, None, None, None, None


def kd_ce_loss(s, t, labels, temp: float, w_ce: float, w_kd: float, row_mask=None) -> torch.Tensor:
    """``w_ce * sum CE(s, label) + w_kd * T^2 * sum KL(softmax(t/T) || softmax(s/T))`` over rows
    (weights carry the normalisation); labels < 0 are ignored for the CE term."""
    return _KdCe.apply(s, t, labels, row_mask, temp, w_ce, w_kd)


def kd_soft_target_loss(s, t, labels, temp: float, w_ce: float = 1.0, w_kd: float = 1.0) -> torch.Tensor:
    """``w_ce * CE(s, labels) + w_kd * T^2 * KL(softmax(t/T) || softmax(s/T))``, both batch means."""
    n = s.shape[0]
    return kd_ce_loss(s, t, labels, temp, w_ce / n, w_kd / n)


def cross_entropy(s, labels) -> torch.Tensor:
    n = s.reshape(-1, s.shape[-1]).shape[0]
    return kd_ce_loss(s, None, labels, 1.0, 1.0 / n, 0.0)


class _Cosine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, row_mask, scale):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y2 = y.detach().reshape(-1, y.shape[-1]).to(x2.dtype).contiguous()
        n, d = x2.shape
        loss = torch.zeros((), dtype=torch.float32, device=x.device)
        gx = torch.empty_like(x2)
        msk = None if row_mask is None else row_mask.reshape(-1).to(torch.uint8).contiguous()
        with on_device(x.device):
            _check(lib().tsp_cosine_loss(_ptr(x2), _ptr(y2), _ptr(msk), _c.c_int(n), _c.c_int(d), _c.c_int(_dt(x2)),
                                         _c.c_float(scale), _ptr(loss), _ptr(gx), _stream()), "tsp_cosine_loss")
        _count()
        ctx.save_for_backward(gx)
        ctx.shape = x.shape
        return loss

    @staticmethod
    def backward(ctx, gout):
        (gx,) = ctx.saved_tensors
        return (gx * gout.to(gx.dtype)).view(ctx.shape), None, None, None


def cosine_embedding_loss(x, y, scale: float, row_mask=None) -> torch.Tensor:
    return _Cosine.apply(x, y, row_mask, scale)


def info_nce_loss(q: torch.Tensor, k: torch.Tensor, temp: float) -> torch.Tensor:
    """InfoNCE of MoCo-v3: ``CE(normalize(q) @ normalize(k)^T / T, arange(N)) * 2T``."""
    from . import gemm
    return gemm.info_nce(q, k, temp)


# ---------------------------------------------------------------------------------------------
# LayerNorm / GELU
# ---------------------------------------------------------------------------------------------
class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        d = x.shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        wf, bf = w.detach().float().contiguous(), b.detach().float().contiguous()
        with on_device(x.device):
            _check(lib().tsp_layernorm_fwd(_ptr(x2), _ptr(wf), _ptr(bf), _ptr(y), _ptr(mean), _ptr(rstd),
                                           _c.c_int(rows), _c.c_int(d), _c.c_float(eps), _c.c_int(_dt(x2)), _stream()),
                   "tsp_layernorm_fwd")
        _count()
        ctx.save_for_backward(x2, wf, mean, rstd)
        ctx.shape = x.shape
        ctx.wdtype = w.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, wf, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d).to(x2.dtype).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty(d, dtype=torch.float32, device=x2.device)
        db = torch.empty(d, dtype=torch.float32, device=x2.device)
        nb = lib().tsp_layernorm_bwd_blocks(_c.c_int(rows))
        partial = torch.empty(nb * 2 * d, dtype=torch.float32, device=x2.device)
        with on_device(x2.device):
            _check(lib().tsp_layernorm_bwd(_ptr(dy2), _ptr(x2), _ptr(wf), _ptr(mean), _ptr(rstd), _ptr(dx), _ptr(dw),
                                           _ptr(db), _ptr(partial), _c.c_int(rows), _c.c_int(d), _c.c_int(_dt(x2)),
                                           _stream()), "tsp_layernorm_bwd")
        _count(3)
        return dx.view(ctx.shape), dw.to(ctx.wdtype), db.to(ctx.wdtype), None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    d = x.shape[-1]
    if not x.is_cuda or d % 8 != 0 or d > 1024 or x.dtype not in (torch.float32, torch.bfloat16):
        return torch.nn.functional.layer_norm(x, (d,), weight, bias, eps)
    return _LayerNorm.apply(x, weight, bias, eps)


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        x = x.contiguous()
        d = x.shape[-1]
        y = torch.empty_like(x)
        bf = None if bias is None else bias.detach().float().contiguous()
        with on_device(x.device):
            _check(lib().tsp_gelu_fwd(_ptr(x), _ptr(bf), _ptr(y), _c.c_int64(x.numel()), _c.c_int(d), _c.c_int(_dt(x)),
                                      _stream()), "tsp_gelu_fwd")
        _count()
        ctx.save_for_backward(x, bf if bf is not None else x.new_empty(0))
        ctx.has_bias = bias is not None
        ctx.bdtype = None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, bf = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        d = x.shape[-1]
        with on_device(x.device):
            _check(lib().tsp_gelu_bwd(_ptr(dy), _ptr(x), _ptr(bf if ctx.has_bias else None), _ptr(dx),
                                      _c.c_int64(x.numel()), _c.c_int(d), _c.c_int(_dt(x)), _stream()), "tsp_gelu_bwd")
        _count()
        db = dx.reshape(-1, d).sum(0).to(ctx.bdtype) if ctx.has_bias else None
        return dx, db


def gelu(x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gelu(x + bias)`` (erf form)."""
    if not x.is_cuda or x.numel() % 8 != 0 or x.dtype not in (torch.float32, torch.bfloat16) or \
            (bias is not None and x.shape[-1] % 8 != 0):
        return torch.nn.functional.gelu(x if bias is None else x + bias)
    return _Gelu.apply(x, bias)


# ---------------------------------------------------------------------------------------------
# data-parallel reduce-scatter + sharded step + all-gather over peer-mapped buffers (csrc/peer.cu)
# ---------------------------------------------------------------------------------------------
@torch.no_grad()
def dp_reduce_norms_(grad_ptrs, n_peers, scale, g_out, p, chunks, seg_hp, norms) -> None:
    L = lib()
    L.tsp_dp_reduce_norms.restype = _c.c_int
    with on_device(p.device):
        _check(L.tsp_dp_reduce_norms(grad_ptrs, _c.c_int(n_peers), _c.c_float(scale), _ptr(g_out), _ptr(p),
                                     _ptr(chunks), _c.c_int(chunks.shape[0]), _ptr(seg_hp), _ptr(norms),
                                     _c.c_int(seg_hp.shape[0]), _stream()), "tsp_dp_reduce_norms")
    _count(2)


@torch.no_grad()
def publish_norms_(table_ptrs, n_peers, self_idx, norms) -> None:
    """This rank's partial LARS norms into slot ``self_idx`` of every replica's table (peer stores)."""
    L = lib()
    L.tsp_publish_norms.restype = _c.c_int
    with on_device(norms.device):
        _check(L.tsp_publish_norms(table_ptrs, _c.c_int(n_peers), _c.c_int(self_idx), _ptr(norms),
                                   _c.c_int(norms.numel()), _stream()), "tsp_publish_norms")
    _count()


@torch.no_grad()
def sum_norms_(table, n_peers, norms) -> None:
    """``norms = sum_r table[r]`` over the replicas' slots."""
    L = lib()
    L.tsp_sum_norms.restype = _c.c_int
    with on_device(norms.device):
        _check(L.tsp_sum_norms(_ptr(table), _c.c_int(n_peers), _c.c_int(norms.numel()), _ptr(norms), _stream()),
               "tsp_sum_norms")
    _count()


@torch.no_grad()
def dp_lars_apply_(param_ptrs, n_peers, self_idx, g, mu, chunks, seg_hp, norms) -> None:
    L = lib()
    L.tsp_dp_lars_apply.restype = _c.c_int
    with on_device(g.device):
        _check(L.tsp_dp_lars_apply(param_ptrs, _c.c_int(n_peers), _c.c_int(self_idx), _ptr(g), _ptr(mu), _ptr(chunks),
                                   _c.c_int(chunks.shape[0]), _ptr(seg_hp), _ptr(norms), _stream()),
               "tsp_dp_lars_apply")
    _count()


@torch.no_grad()
def dp_adamw_step_(grad_ptrs, param_ptrs, n_peers, self_idx, scale, m, v, chunks, seg_hp) -> None:
    L = lib()
    L.tsp_dp_adamw_step.restype = _c.c_int
    with on_device(m.device):
        _check(L.tsp_dp_adamw_step(grad_ptrs, param_ptrs, _c.c_int(n_peers), _c.c_int(self_idx), _c.c_float(scale),
                                   _ptr(m), _ptr(v), _ptr(chunks), _c.c_int(chunks.shape[0]), _ptr(seg_hp),
                                   _stream()), "tsp_dp_adamw_step")
    _count()
