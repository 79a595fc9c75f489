"""Stage-boundary links over peer-mapped memory: copy engines move the bytes, one-thread kernels order them.

A pipeline stage's compute kernels are persistent grids that want every SM.  A library send / receive pair is a
kernel of several thread blocks on each side that stays resident while it waits for its partner, so every
convolution launched meanwhile runs with some of its blocks queued behind it.  This link keeps the SMs out of the
transfer:

* the RECEIVER owns a ring of ``slots`` message slots (one device buffer, exported once through CUDA IPC) and a
  sequence word; the SENDER owns an acknowledgement word;
* ``send`` (on a private stream, ordered after the caller's stream): wait - bounded, one thread - until the slot of
  message ``q`` has been released (``ack >= q - slots + 1``), copy the tensors into the slot with the copy engine
  (``csrc/peer.cu: tsp_copy_async``, a peer write over NVLink), then store ``q + 1`` into the receiver's sequence word
  with release semantics (``tsp_signal_arrive``);
* ``post_recv`` (on the receiver's private stream, ahead of time): wait - bounded, one thread - for the sequence word
  to reach ``q + 1``, copy the slot into freshly allocated tensors, and store ``q + 1`` into the sender's
  acknowledgement word.  The compute stream later waits on the event behind that copy.

The slot size follows the largest message seen: when a message does not fit, both sides (which see the same tensor
specs in the same order) open a new epoch; the receiver allocates a larger ring and publishes its handle in the
rendezvous store, the sender maps it.  Every device-side wait gives up after ``limit_ms``, records a code in the
link's status word and lets the stream continue; :meth:`PeerLink.poll` raises on the host.

Same interface as :class:`tspipe_b200.comm.links.Link` (the ``torch.distributed`` p2p link, which stays the path
for CPU ranks, for ranks on different nodes and for GPUs without a peer path).  The reference negotiates every
transfer by RPC and synchronises the device around a locked ``dist.send`` / ``dist.recv``
(`tspipe/communicator.py:570-678`).
"""
from __future__ import annotations

import ctypes as _c
import pickle
from typing import Any, List, Optional, Sequence, Tuple

import torch

from . import peer
from .links import RecvHandle, TensorSpec, wire_empty, wire_form

_ALIGN = 256


class LinkTimeout(RuntimeError):
    pass


class _EventWork:
    """What :class:`RecvHandle` needs from a work object: make the current stream wait for the data."""
    __slots__ = ("event",)

    def __init__(self, event):
        self.event = event

    def wait(self) -> None:
        torch.cuda.current_stream().wait_event(self.event)

    def is_completed(self) -> bool:
        return self.event.query()


def _nbytes(shape: Sequence[int], dtype: torch.dtype) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n * torch.empty((), dtype=dtype).element_size()


def _layout(specs: Sequence[TensorSpec]) -> Tuple[List[int], int]:
    """Byte offset of every tensor inside a slot (256-byte aligned) and the slot bytes needed."""
    offs, pos = [], 0
    for shape, dtype in specs:
        offs.append(pos)
        pos += -(-_nbytes(shape, dtype) // _ALIGN) * _ALIGN
    return offs, max(pos, _ALIGN)


class PeerLink:
    """One direction of one stage boundary over peer memory; a rank only ever sends or only ever receives on it."""

    SEND_WAIT, RECV_WAIT = 21, 22
    _instances: dict = {}

    def __init__(self, store, name: str, device: torch.device, slots: int = 4, limit_ms: int = 120000,
                 channels_last: bool = False):
        from ..ops import fused
        self.channels_last = bool(channels_last)
        # links of the same name made one after the other in a process (several pipelines over one process group)
        # get store keys of their own; both ends create their links in the same order
        n = PeerLink._instances.get(name, 0)
        PeerLink._instances[name] = n + 1
        self.store, self.name, self.device = store, f"{name}#{n}", device
        self.slots, self.limit_ms = max(int(slots), 1), int(limit_ms)
        self.cuda = True
        self.stream = torch.cuda.Stream(device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_event: Optional[torch.cuda.Event] = None
        self._seq = 0                 # next message number (both sides count the same messages)
        self._epoch, self._cap, self._first = 0, 0, 0
        self._word: Optional[torch.Tensor] = None      # the word this side owns (sender: ack, receiver: sequence)
        self._remote_word = None      # pointer table with the peer's word
        self._ring: Optional[torch.Tensor] = None      # receiver: current ring
        self._old_rings: List[torch.Tensor] = []
        self._ring_ptr = 0            # sender: mapped base of the receiver's ring
        L = fused.lib()
        for fn in ("tsp_signal_arrive", "tsp_signal_wait", "tsp_copy_async"):
            getattr(L, fn).restype = _c.c_int
        self._lib = L

    # -- rendezvous ----------------------------------------------------------------------------------
    def _publish(self, key: str, tensor: torch.Tensor, **extra) -> None:
        handle, offset = peer._export(tensor)
        self.store.set(f"{self.name}/{key}", pickle.dumps(dict(handle=handle, offset=offset, **extra)))

    def _map(self, key: str) -> Tuple[int, dict]:
        info = pickle.loads(self.store.get(f"{self.name}/{key}"))
        with torch.cuda.device(self.device):
            h = info["handle"]
            if h not in peer._open_handles:
                peer._open_handles[h] = peer._import(h)
        return peer._open_handles[h] + info["offset"], info

    def _own_word(self, key: str, peer_key: str) -> None:
        """First use: create and publish this side's word, map the peer's."""
        if self._word is not None:
            return
        self._word = torch.zeros(8, dtype=torch.int32, device=self.device)
        torch.cuda.current_stream().synchronize()          # the zeros are in memory before the peer can write
        self._publish(key, self._word)
        ptr, _ = self._map(peer_key)
        table = (_c.c_void_p * 1)()
        table[0] = ptr
        self._remote_word = table

    # -- device-side pieces --------------------------------------------------------------------------
    def _wait(self, value: int, code: int) -> None:
        from ..ops import fused
        fused._check(self._lib.tsp_signal_wait(fused._ptr(self._word), _c.c_int(1), _c.c_int(value),
                                               _c.c_int(self.limit_ms), fused._ptr(self.status), _c.c_int(code),
                                               fused._stream()), "tsp_signal_wait")
        fused._count()

    def _arrive(self, value: int) -> None:
        from ..ops import fused
        fused._check(self._lib.tsp_signal_arrive(self._remote_word, _c.c_int(1), _c.c_int(0), _c.c_int(value),
                                                 fused._stream()), "tsp_signal_arrive")
        fused._count()

    # -- send ----------------------------------------------------------------------------------------
    def send(self, tensors: Sequence[torch.Tensor]) -> None:
        """Enqueue the transfer of ``tensors`` (one message), ordered after the work already queued on the current
        stream.  Blocks the host only when the receiver has to publish a larger ring first."""
        from ..ops import fused
        tensors = [wire_form(t, self.channels_last) for t in tensors]
        offs, need = _layout([(tuple(t.shape), t.dtype) for t in tensors])
        q = self._seq
        self._seq += 1
        self._own_word("ack", "seq")
        if need > self._cap:
            self._epoch += 1
            self._ring_ptr, info = self._map(f"ring/{self._epoch}")
            self._cap, self._first = int(info["slot_bytes"]), q
            assert self._cap >= need and int(info["first"]) == q, "the two ends of the link disagree on the messages"
        slot = self._ring_ptr + ((q - self._first) % self.slots) * self._cap
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            if q >= self.slots:
                self._wait(q - self.slots + 1, self.SEND_WAIT)
            st = fused._stream()
            for t, off in zip(tensors, offs):
                t.record_stream(self.stream)
                fused._check(self._lib.tsp_copy_async(_c.c_void_p(slot + off), fused._ptr(t),
                                                      _c.c_int64(t.numel() * t.element_size()), st), "tsp_copy_async")
            self._arrive(q + 1)

    def flush(self) -> None:
        self.stream.synchronize()
        self.poll(sync=True)

    # -- receive -------------------------------------------------------------------------------------
    def post_recv(self, specs: Sequence[TensorSpec]) -> RecvHandle:
        specs = [(tuple(shape), dtype) for shape, dtype in specs]
        offs, need = _layout(specs)
        q = self._seq
        self._seq += 1
        if need > self._cap:
            self._epoch += 1
            cap = -(-need // (1 << 20)) * (1 << 20)
            with torch.cuda.stream(self.stream):
                ring = torch.empty(self.slots * cap, dtype=torch.uint8, device=self.device)
            if self._ring is not None:
                self._old_rings.append(self._ring)        # messages of the old epoch may still be in flight
            self._ring, self._cap, self._first = ring, cap, q
            self._publish(f"ring/{self._epoch}", ring, slot_bytes=cap, first=q)
        self._own_word("seq", "ack")
        base = ((q - self._first) % self.slots) * self._cap
        with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
            self._wait(q + 1, self.RECV_WAIT)
            bufs = []
            for (shape, dtype), off in zip(specs, offs):
                n = _nbytes(shape, dtype)
                buf, b = wire_empty(shape, dtype, self.device, self.channels_last)
                if n:
                    buf.view(-1).view(torch.uint8).copy_(self._ring[base + off: base + off + n])
                bufs.append(b)
            self._arrive(q + 1)
            done = torch.cuda.Event()
            done.record()
        return RecvHandle(bufs, [_EventWork(done)], self.stream)

    # -- errors --------------------------------------------------------------------------------------
    def poll(self, sync: bool = False) -> None:
        """Raise :class:`LinkTimeout` when a device-side wait of this link gave up.  Without ``sync`` the check is
        one step late: it looks at the copy of the status word started by the previous call."""
        if sync:
            code = int(self.status.item())
        else:
            code = 0
            if self._status_event is not None and self._status_event.query():
                code = int(self._status_host[0])
                self._status_event = None
            if self._status_event is None:
                with torch.cuda.stream(self.stream):
                    self._status_host.copy_(self.status, non_blocking=True)
                    self._status_event = torch.cuda.Event()
                    self._status_event.record()
        if code:
            side = "sender waited for a free slot" if code == self.SEND_WAIT else "receiver waited for a message"
            raise LinkTimeout(f"link {self.name}: {side} longer than {self.limit_ms} ms")


def make_link(group, peer_rank: int, device: torch.device, store=None, name: str = "", peer_device: Optional[int] = None,
              use_peer: bool = True, slots: int = 4, limit_ms: int = 120000, channels_last: bool = False):
    """:class:`PeerLink` when both ends are CUDA devices of this node with a peer path, else the
    ``torch.distributed`` :class:`~tspipe_b200.comm.links.Link`.  Both ends evaluate the same condition."""
    from .links import Link
    if (use_peer and device.type == "cuda" and store is not None and peer_device is not None
            and peer_device != device.index and torch.cuda.can_device_access_peer(device.index, peer_device)):
        return PeerLink(store, name, device, slots=slots, limit_ms=limit_ms, channels_last=channels_last)
    return Link(group, peer_rank, device, channels_last=channels_last)
