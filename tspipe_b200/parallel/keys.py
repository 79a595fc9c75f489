"""Cross-replica all-gather of MoCo keys.

DDP baseline of the reference: ``concat_all_gather`` (NCCL all-gather without gradient) and labels offset
by rank (`benchmarks/moco-v3/moco/builder.py:73-85,138-149`); its pipeline mode drops the gather because
one pipeline sees the whole batch (`benchmarks/moco-v3/main.py:154,159`).  With ``R`` pipeline replicas the
loss stage of every replica holds ``N/R`` keys.  Peer path: each loss-stage rank keeps two key slots mapped
into its peers; a step writes the local keys into the slot of its parity, a stream-ordered tiny collective
marks "everyone has written", and one kernel (``tsp_gather_blocks``) pulls all ``R`` blocks with peer
loads into the local ``[N, D]`` key matrix that feeds the contrastive-logit GEMM through TMA.  Two slots
make the "everyone has read" barrier unnecessary: a slot is rewritten two steps later, after the next
step's barrier.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..runtime import context


def gather_keys(k: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """``(k_all [N, D], label_offset)`` for the replica this rank belongs to; identity without replicas."""
    ctx = context.current()
    if ctx is None or ctx.topo.dp <= 1:
        return k, 0
    topo = ctx.topo
    n = k.shape[0]
    k = k.detach().contiguous()
    if not (k.is_cuda and ctx.peer_memory and ctx.fused and (k.numel() * k.element_size()) % 16 == 0):
        parts = [torch.empty_like(k) for _ in range(topo.dp)]
        dist.all_gather(parts, k, group=topo.dp_group)
        return torch.cat(parts), n * topo.replica
    from ..comm import peer
    from ..ops import fused
    key = ("moco_keys", tuple(k.shape), k.dtype)
    st = ctx.cache.get(key)
    if st is None:
        slots = [torch.zeros_like(k) for _ in range(2)]
        views = [peer.exchange(s, topo.dp_group, topo.dp_ranks) for s in slots]
        st = ctx.cache[key] = dict(slots=slots, tables=[peer.pointer_table(v) for v in views], keep=views, step=0,
                                   token=torch.zeros(1, device=k.device))
    par = st["step"] & 1
    st["step"] += 1
    st["slots"][par].copy_(k)
    dist.all_reduce(st["token"], group=topo.dp_group)         # all replicas' keys of this step are in place
    out = torch.empty((topo.dp * n,) + tuple(k.shape[1:]), dtype=k.dtype, device=k.device)
    L = fused.lib()
    L.tsp_gather_blocks.restype = ctypes.c_int
    with torch.cuda.device(k.device):
        fused._check(L.tsp_gather_blocks(st["tables"][par], ctypes.c_int(topo.dp),
                                         ctypes.c_int64(k.numel() * k.element_size()), fused._ptr(out),
                                         fused._stream()), "tsp_gather_blocks")
    fused._count()
    return out, n * topo.replica
