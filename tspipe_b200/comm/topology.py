"""Rank layout and process groups.

The reference runs one pipeline over all GPUs plus a scheduler rank, with TensorPipe RPC
for control and one NCCL group for tensors (`tspipe/tspipe.py:94`,
`tspipe/communicator.py:422-464`).  Here every rank is a GPU (or CPU) worker laid out as a
``dp x pp`` grid (``rank = replica * pp + stage``); there is no scheduler rank because
each worker derives its own column of the schedule.  Each stage boundary gets two
two-rank groups - one per direction - so that forward activations and backward gradients
never share an NCCL stream (a receive posted early for one direction must not block a send
in the other).  Same-stage ranks of all replicas form the data-parallel group.  The
rendezvous key-value store doubles as the control plane.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


@dataclass
class Topology:
    world: int
    rank: int
    pp: int
    dp: int
    backend: str = "gloo"
    device: torch.device = torch.device("cpu")
    fwd_groups: Dict[int, object] = field(default_factory=dict)   # boundary j (between stage j and j+1)
    bwd_groups: Dict[int, object] = field(default_factory=dict)
    dp_group: Optional[object] = None
    pp_group: Optional[object] = None
    store: Optional[object] = None

    def __post_init__(self):
        if self.pp * self.dp != self.world:
            raise ValueError(f"world size {self.world} != dp {self.dp} x pp {self.pp}")

    @property
    def stage(self) -> int:
        return self.rank % self.pp

    @property
    def replica(self) -> int:
        return self.rank // self.pp

    def rank_of(self, replica: int, stage: int) -> int:
        return replica * self.pp + stage

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.pp - 1

    @property
    def prev_rank(self) -> Optional[int]:
        return None if self.is_first else self.rank - 1

    @property
    def next_rank(self) -> Optional[int]:
        return None if self.is_last else self.rank + 1

    @property
    def dp_ranks(self) -> List[int]:
        return [self.rank_of(r, self.stage) for r in range(self.dp)]

    @property
    def is_cuda(self) -> bool:
        return self.device.type == "cuda"


def init_distributed(rank: int, world: int, backend: str, master_addr: str, master_port: int,
                     device: torch.device, timeout_s: float = 600.0) -> None:
    """Join the default process group (no-op if the launcher already did)."""
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", master_addr)
    os.environ.setdefault("MASTER_PORT", str(master_port))
    kwargs = {}
    if backend == "nccl":
        torch.cuda.set_device(device)
        kwargs["device_id"] = device
    dist.init_process_group(backend=backend, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kwargs)


_instances = 0


def build_topology(pp: int, dp: int, device: torch.device, backend: Optional[str] = None,
                   timeout_s: float = 600.0) -> Topology:
    """Create every subgroup.  All ranks call this collectively, in the same order."""
    assert dist.is_initialized()
    world, rank = dist.get_world_size(), dist.get_rank()
    backend = backend or dist.get_backend()
    topo = Topology(world=world, rank=rank, pp=pp, dp=dp, backend=backend, device=device)
    to = datetime.timedelta(seconds=timeout_s)
    for r in range(dp):
        for j in range(pp - 1):
            pair = [topo.rank_of(r, j), topo.rank_of(r, j + 1)]
            gf = dist.new_group(ranks=pair, timeout=to)
            gb = dist.new_group(ranks=pair, timeout=to)
            if rank in pair:
                topo.fwd_groups[j] = gf
                topo.bwd_groups[j] = gb
    for r in range(dp):
        ranks = [topo.rank_of(r, j) for j in range(pp)]
        if pp > 1:
            g = dist.new_group(ranks=ranks, timeout=to)
            if rank in ranks:
                topo.pp_group = g
    if dp > 1:
        for j in range(pp):
            ranks = [topo.rank_of(r, j) for r in range(dp)]
            g = dist.new_group(ranks=ranks, timeout=to)
            if rank in ranks:
                topo.dp_group = g
    from torch.distributed.distributed_c10d import _get_default_store
    global _instances
    _instances += 1             # every TSPipe instance of a job gets its own key space in the store
    topo.store = dist.PrefixStore(f"tspipe_ctl{_instances}", _get_default_store())
    return topo
