"""What a loss function may ask the runtime while it runs on the loss stage: the rank layout (for
cross-replica terms such as MoCo's key all-gather) and whether the fused kernels are on."""
from __future__ import annotations

import threading
from typing import Optional

_tls = threading.local()


class RuntimeContext:
    def __init__(self, topo, fused: bool, peer_memory: bool):
        self.topo, self.fused, self.peer_memory = topo, fused, peer_memory
        self.cache = {}


def set_current(ctx: Optional[RuntimeContext]) -> None:
    _tls.ctx = ctx


def current() -> Optional[RuntimeContext]:
    return getattr(_tls, "ctx", None)
