"""Peer-mapped device buffers: other ranks' buffers addressable by this rank's kernels.

Every GPU of a B200 node reaches every other through NVSwitch at full NVLink 5 bandwidth, so a
kernel can simply load from / store to a neighbour's buffer once it is mapped.  A buffer is exported
as a CUDA IPC handle of its allocation plus a byte offset, the handles travel through an object
collective of the group, and every rank maps its peers' allocations **with its own device current**
(``csrc/peer.cu: tsp_ipc_import``), which is what makes the pointer valid inside its kernels.
(CUDA IPC rule: a mapping is usable by kernels of the device that was current when the handle was opened.  A
mapping opened under the *owner's* device ordinal - what ``torch.multiprocessing``'s tensor rebuilding does -
serves library copies but faults when a kernel of another device dereferences it.)  Peers appear as :class:`PeerView` objects: pointer + length, sliceable,
accepted by the kernel bindings wherever a flat tensor is.

The reference moves every such byte with an RPC-negotiated ``dist.send/recv`` pair
(`tspipe/communicator.py:570-678`) and keeps all parameter exchange on the owning GPU.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Union

import torch
import torch.distributed as dist


class PeerView:
    """A contiguous 1-D range of another GPU's memory, mapped into this process.  Duck-types the few
    tensor methods the kernel bindings use."""

    def __init__(self, ptr: int, numel: int, dtype: torch.dtype, owner_rank: int, keep=None):
        self._ptr, self._numel, self.dtype, self.owner_rank, self._keep = ptr, numel, dtype, owner_rank, keep
        self._esize = torch.empty((), dtype=dtype).element_size()

    def data_ptr(self) -> int:
        return self._ptr

    def numel(self) -> int:
        return self._numel

    def is_contiguous(self) -> bool:
        return True

    def __len__(self) -> int:
        return self._numel

    def __getitem__(self, sl: slice) -> "PeerView":
        start, stop, step = sl.indices(self._numel)
        assert step == 1
        return PeerView(self._ptr + start * self._esize, max(stop - start, 0), self.dtype, self.owner_rank, self)


class _Mapping:
    def __init__(self, base: int):
        self.base = base


def enable_peer_access(peer_device: int) -> None:
    from ..ops import fused
    L = fused.lib()
    L.tsp_enable_peer_access.restype = ctypes.c_int
    code = L.tsp_enable_peer_access(ctypes.c_int(peer_device))
    if code != 0:
        raise RuntimeError(f"no peer access from cuda:{torch.cuda.current_device()} to cuda:{peer_device} (code {code})")


def _export(tensor: torch.Tensor):
    """(ipc handle bytes, byte offset of ``tensor`` inside the exported allocation)."""
    st = tensor.untyped_storage()
    info = st._share_cuda_()
    handle, off_bytes = bytes(info[1]), info[3]
    if len(handle) == 66:
        # recent allocators prefix the 64-byte cudaIpcMemHandle_t with a version byte and a kind byte
        # ('c' = plain cudaMalloc block, 'e' = expandable segment, which legacy IPC cannot export)
        if handle[1:2] != b"c":
            raise RuntimeError("peer mapping needs cudaMalloc-backed allocations (expandable_segments must be off)")
        handle = handle[2:]
    if len(handle) != 64:
        raise RuntimeError(f"unexpected CUDA IPC handle length {len(handle)}")
    return handle, int(off_bytes) + tensor.storage_offset() * tensor.element_size()


def _import(handle: bytes) -> int:
    from ..ops import fused
    L = fused.lib()
    L.tsp_ipc_import.restype = ctypes.c_int
    base = ctypes.c_void_p(0)
    buf = (ctypes.c_ubyte * 64).from_buffer_copy(handle[:64])
    code = L.tsp_ipc_import(buf, ctypes.byref(base))
    if code != 0:
        raise RuntimeError(f"cudaIpcOpenMemHandle failed with code {code}")
    return int(base.value)


_open_handles: Dict[bytes, int] = {}


def exchange(tensor: torch.Tensor, group, group_ranks: Sequence[int]) -> List[Union[torch.Tensor, PeerView]]:
    """All ranks of ``group`` call this with their own contiguous CUDA tensor (from the caching
    allocator).  Returns one entry per group member in ``group_ranks`` order: this rank's own tensor at its
    position, :class:`PeerView` s of the peers' buffers elsewhere.  Owners must keep their tensors alive
    while peers use them."""
    assert tensor.is_cuda and tensor.is_contiguous()
    me = dist.get_rank()
    handle, offset = _export(tensor)
    gathered: List[Optional[tuple]] = [None] * len(group_ranks)
    dist.all_gather_object(gathered, (handle, offset, tensor.numel(), str(tensor.dtype)), group=group)
    out: List[Union[torch.Tensor, PeerView]] = []
    with torch.cuda.device(tensor.device):
        for r, item in zip(group_ranks, gathered):
            if r == me:
                out.append(tensor)
                continue
            h, off, numel, dt = item
            if h not in _open_handles:          # an allocation may be mapped only once per process
                _open_handles[h] = _import(h)
            dtype = getattr(torch, dt.split(".")[-1])
            out.append(PeerView(_open_handles[h] + off, numel, dtype, r))
    return out


def share_over_group(flat, topo) -> Dict[int, Union[torch.Tensor, PeerView]]:
    """Student flat buffers of all stages of this rank's pipeline replica: ``{stage: buffer}``."""
    ranks = [topo.rank_of(topo.replica, j) for j in range(topo.pp)]
    bufs = exchange(flat.data, topo.pp_group, ranks)
    return {j: t for j, t in enumerate(bufs)}


def pointer_table(buffers: Sequence[Union[torch.Tensor, PeerView]]):
    """Host array of device pointers for the ``void* const*`` arguments of ``csrc/peer.cu``."""
    arr = (ctypes.c_void_p * len(buffers))()
    for i, t in enumerate(buffers):
        arr[i] = t.data_ptr()
    return arr


def multicast_supported(device: Optional[int] = None) -> Optional[bool]:
    """Whether the GPU can join NVLink multicast objects (NVLS, what ``multimem`` instructions address): a capability
    query through the driver, nothing is allocated or bound.  ``None`` when it cannot be asked (no CUDA, old driver).
    The runtime records the answer at start-up; its cross-GPU kernels use peer loads / stores either way."""
    if not torch.cuda.is_available():
        return None
    from ..ops import fused
    L = fused.lib()
    L.tsp_multicast_supported.restype = ctypes.c_int
    code = int(L.tsp_multicast_supported(ctypes.c_int(torch.cuda.current_device() if device is None else device)))
    return None if code < 0 else bool(code)
