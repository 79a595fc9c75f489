"""Stage-boundary tensor links over ``torch.distributed`` point-to-point.

Replaces the reference's channel machinery - metadata RPC, agreement RPC, locked NCCL
send/recv and a device-wide synchronize per transfer (`tspipe/communicator.py:243-308,
570-678`) - with plain ordered p2p on a direction-private communicator:

* the receiver posts its receives ahead of time, in the sender's (schedule-determined)
  order, from an otherwise idle stream, and the compute stream later waits on the
  transfer's completion event - no host synchronisation on either side;
* tensor shapes are announced once per (link, net, shape-epoch) through the key-value
  store, not per message.

On CPU (gloo) the same code runs with host-blocking ``wait``.
"""
from __future__ import annotations

import pickle
from collections import deque
from typing import Any, Deque, Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist

TensorSpec = Tuple[Tuple[int, ...], torch.dtype]


class RecvHandle:
    __slots__ = ("tensors", "works", "_stream", "_done")

    def __init__(self, tensors: List[torch.Tensor], works: List[Any], stream):
        self.tensors, self.works, self._stream, self._done = tensors, works, stream, False

    def wait(self) -> List[torch.Tensor]:
        """Make the *current* stream (or the host, on CPU) wait for the data."""
        if not self._done:
            for w in self.works:
                w.wait()
            if self._stream is not None:
                cur = torch.cuda.current_stream()
                for t in self.tensors:
                    t.record_stream(cur)
            self._done = True
        return self.tensors


def wire_form(t: torch.Tensor, channels_last: bool) -> torch.Tensor:
    """The contiguous tensor whose bytes cross a link for ``t``.  With ``channels_last`` a 4-D tensor travels in NHWC
    order (as an ``[N, H, W, C]`` view when it is already laid out that way - no copy), so that an activation of a
    channels-last network is not transposed on the way out and back again on the way in."""
    if channels_last and t.dim() == 4:
        return t.permute(0, 2, 3, 1).contiguous()          # a view when t is channels-last
    return t if t.is_contiguous() else t.contiguous()


def wire_empty(shape: Sequence[int], dtype: torch.dtype, device, channels_last: bool
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(buffer, tensor)``: the contiguous receive buffer of a tensor of ``shape`` and the tensor the consumer sees
    (the same memory; NCHW-shaped with channels-last strides when ``channels_last`` applies)."""
    if channels_last and len(shape) == 4:
        n, c, h, w = shape
        buf = torch.empty((n, h, w, c), dtype=dtype, device=device)
        return buf, buf.permute(0, 3, 1, 2)
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    return buf, buf


class Link:
    """One direction of one stage boundary, as seen from one of its two ranks."""

    def __init__(self, group, peer: int, device: torch.device, channels_last: bool = False):
        self.group, self.peer, self.device = group, peer, device
        self.cuda = device.type == "cuda"
        self.channels_last = bool(channels_last)
        self.post_stream = torch.cuda.Stream(device) if self.cuda else None
        self._pending: Deque[Tuple[List[Any], List[torch.Tensor]]] = deque()

    # -- send ---------------------------------------------------------------------------------
    def send(self, tensors: Sequence[torch.Tensor]) -> None:
        """Enqueue sends ordered after the work already queued on the current stream."""
        tensors = [wire_form(t, self.channels_last) for t in tensors]
        works = [dist.isend(t, self.peer, group=self.group) for t in tensors]
        self._pending.append((works, tensors))
        self._reap()

    def _reap(self) -> None:
        while self._pending and all(w.is_completed() for w in self._pending[0][0]):
            self._pending.popleft()

    def flush(self) -> None:
        while self._pending:
            works, _ = self._pending.popleft()
            for w in works:
                w.wait()

    # -- receive ------------------------------------------------------------------------------
    def post_recv(self, specs: Sequence[TensorSpec]) -> RecvHandle:
        if self.cuda:
            with torch.cuda.stream(self.post_stream):
                pairs = [wire_empty(shape, dtype, self.device, self.channels_last) for shape, dtype in specs]
                works = [dist.irecv(b, self.peer, group=self.group) for b, _ in pairs]
            return RecvHandle([t for _, t in pairs], works, self.post_stream)
        pairs = [wire_empty(shape, dtype, None, self.channels_last) for shape, dtype in specs]
        works = [dist.irecv(b, self.peer, group=self.group) for b, _ in pairs]
        return RecvHandle([t for _, t in pairs], works, None)


class MetaBoard:
    """Structure / shape announcements through the rendezvous store.

    For every ``(link, net, batch)`` the sender publishes once the pytree structure and tensor specs
    of what crosses the link (identical for all microbatches of the batch); the receiver reads the key
    before posting the batch's first receive and deletes it.  The reference ships this metadata with
    every single message by RPC (`tspipe/communicator.py:84-99,251-267`)."""

    def __init__(self, store, replica: int):
        self.store, self.replica = store, replica
        self._sent: Dict[str, bytes] = {}
        self._got: Dict[str, Any] = {}

    def _key(self, link: str, net: str, batch: int) -> str:
        return f"meta/{self.replica}/{link}/{net}/{batch}"

    def publish(self, link: str, net: str, batch: int, meta: Any) -> None:
        key = self._key(link, net, batch)
        blob = pickle.dumps(meta)
        prev = self._sent.get(key)
        if prev is None:
            self.store.set(key, blob)
            self._sent[key] = blob
            for k in [k for k in self._sent if k.endswith(f"/{batch - 4}")]:
                del self._sent[k]
        elif prev != blob:
            raise RuntimeError(f"stage output structure differs between microbatches of batch {batch} on "
                               f"{link}/{net}: all microbatches of a batch must have the same shapes")

    def cached(self, link: str, net: str, batch: int) -> bool:
        key = self._key(link, net, batch)
        if key in self._got:
            return True
        try:
            if not self.store.check([key]):
                return False
        except Exception:
            return False
        self.fetch(link, net, batch)
        return True

    def fetch(self, link: str, net: str, batch: int) -> Any:
        key = self._key(link, net, batch)
        if key not in self._got:
            import warnings
            with warnings.catch_warnings():             # tree specs of older pickles warn about their own class names
                warnings.simplefilter("ignore", FutureWarning)
                self._got[key] = pickle.loads(self.store.get(key))
            try:
                self.store.delete_key(key)
            except Exception:
                pass
            for k in [k for k in self._got if k.endswith(f"/{batch - 4}")]:
                del self._got[k]
        return self._got[key]
