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


class KeyExchange:
    """Two peer-mapped slots per rank for one (shape, dtype) of keys; :meth:`publish` writes this step's
    keys into the slot of the step's parity and returns every replica's slot of that parity once a
    stream-ordered collective has established that all of them are written."""

    def __init__(self, like: torch.Tensor, topo):
        from ..comm import peer
        self.topo = topo
        self.slots = [torch.zeros_like(like) for _ in range(2)]
        self.views = [peer.exchange(s, topo.dp_group, topo.dp_ranks) for s in self.slots]
        self.tables = [peer.pointer_table(v) for v in self.views]
        self.token = torch.zeros(1, device=like.device)
        self.step = 0

    def publish(self, k: torch.Tensor):
        par = self.step & 1
        self.step += 1
        self.slots[par].copy_(k)
        dist.all_reduce(self.token, group=self.topo.dp_group)     # all replicas' keys of this step are in place
        return self.views[par], self.tables[par]


def exchange_for(k: torch.Tensor, tag: str) -> Optional[KeyExchange]:
    ctx = context.current()
    if ctx is None or ctx.topo.dp <= 1 or not (k.is_cuda and ctx.peer_memory and ctx.fused):
        return None
    key = (tag, tuple(k.shape), k.dtype)
    if key not in ctx.cache:
        ctx.cache[key] = KeyExchange(k, ctx.topo)
    return ctx.cache[key]


def gather_blocks(table, n_peers: int, like: torch.Tensor) -> torch.Tensor:
    """Concatenate every replica's block (read with peer loads) into a local ``[R*n, ...]`` tensor."""
    from ..ops import fused
    out = torch.empty((n_peers * like.shape[0],) + tuple(like.shape[1:]), dtype=like.dtype, device=like.device)
    L = fused.lib()
    L.tsp_gather_blocks.restype = ctypes.c_int
    with torch.cuda.device(like.device):
        fused._check(L.tsp_gather_blocks(table, ctypes.c_int(n_peers), ctypes.c_int64(like.numel() * like.element_size()),
                                         fused._ptr(out), fused._stream()), "tsp_gather_blocks")
    fused._count()
    return out


def gather_keys(k: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """``(k_all [N, D], label_offset)`` for the replica this rank belongs to; identity without replicas."""
    ctx = context.current()
    if ctx is None or ctx.topo.dp <= 1:
        return k, 0
    topo = ctx.topo
    n = k.shape[0]
    k = k.detach().contiguous()
    ex = exchange_for(k, "moco_keys") if (k.numel() * k.element_size()) % 16 == 0 else None
    if ex is None:
        parts = [torch.empty_like(k) for _ in range(topo.dp)]
        dist.all_gather(parts, k, group=topo.dp_group)
        return torch.cat(parts), n * topo.replica
    _, table = ex.publish(k)
    return gather_blocks(table, topo.dp, k), n * topo.replica
