"""Bindings of the tcgen05 / TMEM / TMA GEMM (``csrc/gemm_tcgen05.cu``) and the ops built on it.

``matmul_nt(a, b)`` computes ``a @ b.T`` for row-major bf16 ``a [M, K]`` and ``b [N, K]`` with fp32
accumulation in tensor memory, optional fused ``+ bias`` and GELU epilogue.  ``linear`` is the autograd
wrapper used by the transformer blocks and heads: forward on the CTA-pair tcgen05 GEMM, ``dX = dY W`` and
``dW = dY^T X`` on the implicit-GEMM kernels of ``csrc/conv_igemm_tcgen05.cu`` (a linear layer is a 1x1
convolution over its rows: the weight is read in place as MN-major tiles, the weight gradient is added into
the fp32 gradient buffer), the bias gradient on the streaming column-sum kernel.  ``info_nce`` is the MoCo-v3 contrastive loss
(`benchmarks/moco-v3/main.py:147-162`): row-normalised ``q @ k.T / T`` on the tcgen05 kernel followed
by the fused cross-entropy kernel (value + gradient in one launch).

The kernel bounds every barrier wait; a non-zero device status word after a launch means a wait ran
out and the output is invalid - :func:`check_status` raises in that case.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional

import torch
import torch.nn.functional as F

from . import fused as _f

_status = {}


def _status_word(device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device=None) -> None:
    """Synchronising check of the GEMM status word (tests and debugging)."""
    for key, t in _status.items():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"tcgen05 GEMM on {key}: bounded wait ran out in role {code} "
                               "(1 = TMA producer, 2 = MMA issuer, 3 = epilogue, 4 = MMA issuer on a free accumulator)")


def eligible(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Shapes and dtypes the tcgen05 linear path takes: bf16 compute (a bf16 input, or bf16 autocast), feature counts
    multiples of 64, at least one full tile of rows."""
    k = x.shape[-1]
    if not (x.is_cuda and weight.is_cuda and weight.dim() == 2):
        return False
    if not (x.dtype == torch.bfloat16 or (torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16)):
        return False
    return k % 64 == 0 and weight.shape[0] % 64 == 0 and x.numel() // k >= 128 and weight.stride(1) == 1 \
        and weight.stride(0) == k


_two_cta = True     # measured faster than the one-CTA kernel on every ViT / head shape tried


def set_two_cta(on: bool) -> None:
    """Route :func:`matmul_nt` through the two-SM kernel (``cta_group::2``, one 256 x 256 tile per CTA pair)."""
    global _two_cta
    _two_cta = bool(on)


def matmul_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False,
              out_dtype: torch.dtype = torch.bfloat16, two_cta: Optional[bool] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T`` (bf16 operands).  ``two_cta`` picks the CTA-pair kernel for this call
    (default: the module setting, see :func:`set_two_cta`)."""
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    a = a if (a.dtype == torch.bfloat16 and a.is_contiguous()) else a.to(torch.bfloat16).contiguous()
    b = b if (b.dtype == torch.bfloat16 and b.is_contiguous()) else b.to(torch.bfloat16).contiguous()
    m, k = a.shape
    n = b.shape[0]
    c = torch.empty(m, n, dtype=out_dtype, device=a.device)
    bf = None if bias is None else bias.detach().float().contiguous()
    epi = 0 if bias is None else (2 if gelu else 1)
    if gelu and bias is None:
        bf, epi = torch.zeros(n, dtype=torch.float32, device=a.device), 2
    L = _f.lib()
    fn = L.tsp_gemm_bf16_tn_2cta if (_two_cta if two_cta is None else two_cta) else L.tsp_gemm_bf16_tn
    fn.restype = _c.c_int
    with _f.on_device(a.device):
        code = fn(_f._ptr(a), _f._ptr(b), _f._ptr(c), _f._ptr(bf), _c.c_int(m), _c.c_int(n), _c.c_int(k),
                  _c.c_int(k), _c.c_int(k), _c.c_int(n), _c.c_int(_f._dt(c)), _c.c_int(epi),
                  _f._ptr(_status_word(a.device)), _f._stream())
    _f._check(code, "tsp_gemm_bf16_tn")
    _f._count()
    return c


_W16 = {}        # id(parameter) -> (parameter, version, bf16 copy); dropped at every optimizer step


def clear_weight_cache() -> None:
    _W16.clear()
    _W16T.clear()


def _w16(weight: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a weight matrix, cast once per parameter and optimizer step.  A row slice of a parameter (the q / k
    / v blocks of a fused projection) maps to the same slice of the parameter's copy.  The cache entry holds the
    parameter itself, so an address that is reused by another tensor can never alias an old entry."""
    if weight.dtype == torch.bfloat16 and weight.is_contiguous():
        return weight.detach()
    base = weight._base if weight._base is not None else weight
    if not base.is_contiguous() or base.dtype == torch.bfloat16:
        return weight.detach().to(torch.bfloat16).contiguous()
    if _f.IN_CAPTURE:                   # inside a CUDA graph the cast is part of the graph
        return weight.detach().to(torch.bfloat16).contiguous()
    hit = _W16.get(id(base))
    if hit is None or hit[0] is not base or hit[1] != base._version:
        hit = (base, base._version, base.detach().to(torch.bfloat16))
        _W16[id(base)] = hit
    b16 = hit[2]
    if base is weight:
        return b16
    return b16.as_strided(weight.shape, weight.stride(), weight.storage_offset() - base.storage_offset())


_W16T = {}       # id(parameter slice base) -> (weight, version, bf16 transposed copy [K, N])


def _w16_t(weight: torch.Tensor) -> torch.Tensor:
    """bf16 ``weight.T`` as a contiguous ``[K, N]`` matrix (the B operand of ``dX = dY @ W`` on the ``A @ B^T`` GEMM),
    made once per weight and optimizer step."""
    if _f.IN_CAPTURE:
        return weight.detach().to(torch.bfloat16).t().contiguous()
    base = weight._base if weight._base is not None else weight
    key = (id(base), weight.storage_offset(), tuple(weight.shape))
    hit = _W16T.get(key)
    if hit is None or hit[0] is not base or hit[1] != base._version:
        hit = (base, base._version, _w16(weight).t().contiguous())
        _W16T[key] = hit
    return hit[2]


def _column_sums(dy2: torch.Tensor) -> torch.Tensor:
    """fp32 column sums of a bf16 matrix (the bias gradient) on the streaming statistics kernel."""
    m, n = dy2.shape
    if n % 8 or n > 4096 or m < 2:
        return dy2.float().sum(0)
    sums = torch.empty(2 * n, dtype=torch.float32, device=dy2.device)
    L = _f.lib()
    L.tsp_bn_stats.restype = _c.c_int
    with _f.on_device(dy2.device):
        _f._check(L.tsp_bn_stats(_f._ptr(dy2), _c.c_int64(m), _c.c_int(n), _c.c_int(_f._dt(dy2)), _f._ptr(sums),
                                 _c.c_int(1), _f._stream()), "tsp_bn_stats")
    _f._count(2)
    return sums[:n]


# dX = dY @ W: on the CTA-pair GEMM against a cached transposed bf16 copy of W (True), or on the implicit-GEMM
# data-gradient kernel that reads W in place as MN-major tiles (False; no transposed copy, about half the speed)
_DX_ON_PAIR_GEMM = True


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16 or not x2.is_contiguous():
            x2 = x2.to(torch.bfloat16).contiguous()
        y = matmul_nt(x2, _w16(weight), bias)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.in_shape = x.shape
        ctx.dtypes = (x.dtype, weight.dtype, None if bias is None else bias.dtype)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import conv as _conv
        x2, weight = ctx.saved_tensors
        m, k = x2.shape
        n = weight.shape[0]
        dy2 = dy.reshape(-1, n)
        if dy2.dtype != torch.bfloat16 or not dy2.is_contiguous():
            dy2 = dy2.to(torch.bfloat16).contiguous()
        L = _conv._lib()
        status = _f._ptr(_status_word(x2.device))
        dims = (_c.c_int(m), _c.c_int(1), _c.c_int(1), _c.c_int(k), _c.c_int(n), _c.c_int(1), _c.c_int(1))
        dx = dw = db = None
        with _f.on_device(x2.device):
            st = _f._stream()
            if ctx.needs_input_grad[0]:
                if _DX_ON_PAIR_GEMM:
                    dx2 = matmul_nt(dy2, _w16_t(weight))          # dX = dY @ W on the CTA-pair GEMM
                else:
                    dx2 = torch.empty((m, k), dtype=torch.bfloat16, device=x2.device)
                    _f._check(L.tsp_conv_dgrad(_f._ptr(dy2), _f._ptr(_w16(weight)), _f._ptr(dx2), *dims, status, st),
                              "tsp_conv_dgrad")
                    _f._count()
                dx = dx2.view(ctx.in_shape)
                if ctx.dtypes[0] != torch.bfloat16:
                    dx = dx.to(ctx.dtypes[0])
            if ctx.needs_input_grad[1]:
                g = weight.grad if weight.is_leaf else None
                if (_conv._ACCUMULATE_IN_PLACE and g is not None and g.dtype == torch.float32 and g.is_contiguous()
                        and g.shape == weight.shape):
                    target = g                     # the kernel adds into the existing gradient buffer
                else:
                    target = torch.zeros((n, k), dtype=torch.float32, device=x2.device)
                    dw = target if weight.dtype == torch.float32 else target.to(weight.dtype)
                _f._check(L.tsp_conv_wgrad(_f._ptr(x2), _f._ptr(dy2), _f._ptr(target), *dims, status, st),
                          "tsp_conv_wgrad")
                _f._count()
                if dw is not None and dw is not target:
                    dw = target.to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _column_sums(dy2).to(ctx.dtypes[2])
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _Linear.apply(x, weight, bias)


def info_nce(q: torch.Tensor, k: torch.Tensor, temp: float, k_all: Optional[torch.Tensor] = None,
             label_offset: int = 0) -> torch.Tensor:
    """``CE(normalize(q) @ normalize(k_all)^T / T, arange(N) + label_offset) * 2T``.  ``k_all`` defaults to
    ``k`` (single replica); with data-parallel replicas it is the concatenation of every replica's keys
    (gathered through peer memory, :func:`tspipe_b200.parallel.keys.gather_keys`)."""
    keys = k if k_all is None else k_all
    qn = F.normalize(q.float(), dim=1)
    kn = F.normalize(keys.detach().float(), dim=1)
    n = q.shape[0]
    if _fused_nce and k_all is None and label_offset == 0 and q.is_cuda and q.shape[1] == 256 and n >= 128:
        return _FusedNCE.apply(qn, kn.to(torch.bfloat16), float(temp))
    if q.is_cuda and q.shape[1] % 8 == 0 and q.shape[1] >= 64 and n >= 128 and keys.shape[0] >= 64:
        logits = _ScaledLogits.apply(qn, kn, 1.0 / temp)
    else:
        logits = qn @ kn.t() / temp
    labels = torch.arange(n, device=q.device) + label_offset
    if q.is_cuda:
        return _f.cross_entropy(logits, labels) * (2 * temp)
    return F.cross_entropy(logits, labels) * (2 * temp)


def matmul_nt_gathered(a: torch.Tensor, b_sources, rows_per_b: int, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``a [M, K] @ concat(b_sources)^T`` where every source is a ``[rows_per_b, K]`` bf16 buffer that may live on
    another GPU (peer-mapped): each CTA pulls its key tile from the owning GPU with its own TMA load."""
    from ..comm.peer import pointer_table
    a = a if (a.dtype == torch.bfloat16 and a.is_contiguous()) else a.to(torch.bfloat16).contiguous()
    m, k = a.shape
    r = len(b_sources)
    c = torch.empty(m, r * rows_per_b, dtype=out_dtype, device=a.device)
    L = _f.lib()
    L.tsp_gemm_bf16_tn_gathered_b.restype = _c.c_int
    with _f.on_device(a.device):
        code = L.tsp_gemm_bf16_tn_gathered_b(_f._ptr(a), pointer_table(b_sources), _c.c_int(r), _c.c_int(rows_per_b),
                                             _f._ptr(c), _c.c_int(m), _c.c_int(k), _c.c_int(k), _c.c_int(k),
                                             _c.c_int(r * rows_per_b), _c.c_int(_f._dt(c)),
                                             _f._ptr(_status_word(a.device)), _f._stream())
    _f._check(code, "tsp_gemm_bf16_tn_gathered_b")
    _f._count()
    return c


class _GatheredLogits(torch.autograd.Function):
    """Contrastive logits against the keys of ALL replicas, read in place from the GPUs that own them."""

    @staticmethod
    def forward(ctx, qn, views, table, rows_per_b, like):
        ctx.table, ctx.r, ctx.like, ctx.adtype = table, len(views), like, qn.dtype
        return matmul_nt_gathered(qn, views, rows_per_b)

    @staticmethod
    def backward(ctx, g):
        from ..parallel.keys import gather_blocks
        k_all = gather_blocks(ctx.table, ctx.r, ctx.like)           # [R*n, D] (already scaled by 1/T)
        return matmul_nt(g, k_all.t().contiguous(), out_dtype=torch.float32).to(ctx.adtype), None, None, None, None


def info_nce_replicas(q: torch.Tensor, k: torch.Tensor, temp: float):
    """InfoNCE across data-parallel replicas with the key all-gather folded into the logit GEMM.  Returns None
    when the fused path does not apply (no replicas, CPU, shapes off the tile grid)."""
    from ..parallel.keys import exchange_for
    from ..runtime import context
    ctx = context.current()
    n, d = q.shape
    if ctx is None or ctx.topo.dp <= 1 or not q.is_cuda or d % 8 or d < 64 or n % 128:
        return None
    if _fused_nce and d == 256 and ctx.topo.dp <= 8:
        # attention-style kernel: every CTA streams key tiles from all replicas' buffers; no logits in memory
        kn16 = F.normalize(k.detach().float(), dim=1).to(torch.bfloat16).contiguous()
        ex = exchange_for(kn16, "moco_keys_bf16")
        if ex is not None:
            views, _ = ex.publish(kn16)
            return _FusedNCEGathered.apply(F.normalize(q.float(), dim=1), kn16, views, float(temp))
    kn = (F.normalize(k.detach().float(), dim=1) * (1.0 / temp)).to(torch.bfloat16).contiguous()
    ex = exchange_for(kn, "moco_keys_scaled_bf16")
    if ex is None:
        return None
    views, table = ex.publish(kn)
    qn = F.normalize(q.float(), dim=1)
    logits = _GatheredLogits.apply(qn, views, table, n, kn)
    labels = torch.arange(n, device=q.device) + n * ctx.topo.replica
    return _f.cross_entropy(logits, labels) * (2 * temp)


_fused_nce = True


def set_fused_nce(on: bool) -> None:
    """Contrastive loss through the fused attention kernel (no N x N logits in memory) when it applies."""
    global _fused_nce
    _fused_nce = bool(on)


_NCE_KEY_SPLIT = True


def set_nce_key_split(flag: bool) -> None:
    """Split the keys of the fused contrastive loss over the grid (default) or run one CTA per query tile."""
    global _NCE_KEY_SPLIT
    _NCE_KEY_SPLIT = bool(flag)


def nce_key_chunks(n_queries: int, n_keys: int, target_ctas: int = 120) -> int:
    """Into how many chunks the fused contrastive loss splits the keys so that (query tiles) x (chunks) fills the
    GPU: the smallest power of two that reaches ``target_ctas`` CTAs, as long as every chunk keeps at least two
    64-row key tiles and the keys divide evenly."""
    if not _NCE_KEY_SPLIT:
        return 1
    tiles = -(-n_queries // 128)
    c = 1
    while tiles * c < target_ctas and n_keys % (2 * c * 64) == 0 and n_keys // (2 * c) >= 128:
        c *= 2
    return c


class _FusedNCE(torch.autograd.Function):
    """``2T * mean_i(logsumexp_j(q_i.k_j / T) - q_i.k_i / T)`` for unit-norm rows, forward and backward from ONE
    pass of the fused attention kernel with V = K: ``lse`` gives the loss, ``O_i = sum_j p_ij k_j`` the gradient
    ``dL/dq_i = 2/N (O_i - k_i)``.  Cosine logits are bounded by 1/T, so the kernel runs without rescaling."""

    @staticmethod
    def forward(ctx, qn, kn16, temp):
        from .attention import flash_fwd
        n, d = qn.shape
        nk = kn16.shape[0]
        q16 = qn.to(torch.bfloat16)
        c = nce_key_chunks(n, nk)
        if c == 1:
            o, lse = flash_fwd(q16.view(1, 1, n, d), kn16.view(1, 1, -1, d), kn16.view(1, 1, -1, d), scale=1.0 / temp,
                               fixed_max=1.0 / temp, out_dtype=torch.float32, want_lse=True)
            o, lse = o.reshape(n, d), lse.view(n)
        else:
            # Keys split over the grid: chunk c of the keys is "head" c of the kernel's (query tile, head) grid, every
            # head sees the same queries.  Each CTA returns its chunk's softmax-weighted key sum and log-sum-exp
            # (exact: the scores are bounded by 1/T, so all chunks use the same fixed maximum); the chunks are then
            # merged with their softmax weights.
            q_rep = q16.unsqueeze(0).expand(c, n, d).contiguous().view(1, c, n, d)
            k_chunks = kn16.view(1, c, nk // c, d)
            o_part, lse_part = flash_fwd(q_rep, k_chunks, k_chunks, scale=1.0 / temp, fixed_max=1.0 / temp,
                                         out_dtype=torch.float32, want_lse=True)
            lse_part = lse_part.view(c, n)
            lse = torch.logsumexp(lse_part, dim=0)
            w = torch.exp(lse_part - lse)                                   # [c, n], sums to 1 over the chunks
            o = torch.einsum("cn,cnd->nd", w, o_part[0])
        pos = (q16.float() * kn16[:n].float()).sum(1) / temp
        ctx.save_for_backward(o, kn16)
        ctx.n, ctx.qdtype = n, qn.dtype
        return (lse - pos).mean() * (2 * temp)

    @staticmethod
    def backward(ctx, g):
        o, kn16 = ctx.saved_tensors
        return ((o - kn16[: ctx.n].float()) * (g * 2.0 / ctx.n)).to(ctx.qdtype), None, None


class _FusedNCEGathered(torch.autograd.Function):
    """:class:`_FusedNCE` against the keys of ALL replicas, read in place from the GPUs that own them (positives
    are the local keys: row i of this replica pairs with key ``i + n * replica`` of the concatenation)."""

    @staticmethod
    def forward(ctx, qn, kn16, views, temp):
        from ..comm.peer import pointer_table
        n, d = qn.shape
        q16 = qn.to(torch.bfloat16).contiguous()
        o = torch.empty(n, d, dtype=torch.float32, device=qn.device)
        lse = torch.empty(n, dtype=torch.float32, device=qn.device)
        L = _f.lib()
        L.tsp_attn_nce_gathered.restype = _c.c_int
        with _f.on_device(qn.device):
            code = L.tsp_attn_nce_gathered(_f._ptr(q16), pointer_table(views), _c.c_int(len(views)), _c.c_int(n),
                                           _f._ptr(o), _f._ptr(lse), _c.c_int(n), _c.c_float(1.0 / temp),
                                           _c.c_float(1.0 / temp), _f._ptr(_status_word(qn.device)), _f._stream())
        _f._check(code, "tsp_attn_nce_gathered")
        _f._count()
        pos = (q16.float() * kn16.float()).sum(1) / temp
        ctx.save_for_backward(o, kn16)
        ctx.n, ctx.qdtype = n, qn.dtype
        return (lse - pos).mean() * (2 * temp)

    @staticmethod
    def backward(ctx, g):
        o, kn16 = ctx.saved_tensors
        return ((o - kn16.float()) * (g * 2.0 / ctx.n)).to(ctx.qdtype), None, None, None


class _ScaledLogits(torch.autograd.Function):
    """``scale * a @ b^T`` in fp32 on the tcgen05 kernel; gradient w.r.t. ``a`` only."""

    @staticmethod
    def forward(ctx, a, b, scale):
        bb = (b * scale).to(torch.bfloat16)
        ctx.save_for_backward(bb)
        ctx.adtype = a.dtype
        return matmul_nt(a.to(torch.bfloat16), bb, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, g):
        (bb,) = ctx.saved_tensors
        # dA = g @ (scale*b): [N, M] x [M, D] -> operands as (g, (scale*b)^T) for the TN kernel
        return matmul_nt(g, bb.t().contiguous(), out_dtype=torch.float32).to(ctx.adtype), None, None
