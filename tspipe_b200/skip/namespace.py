"""Isolation of skip-tensor names (`tspipe/skip/namespace.py:10-43`): two instances of the same
skippable module can stash under the same name without colliding when each is ``isolate``d into
its own :class:`Namespace`."""
from __future__ import annotations

import uuid
from functools import total_ordering
from typing import Any


@total_ordering
class Namespace:
    __slots__ = ("id",)

    def __init__(self) -> None:
        self.id = uuid.uuid4()

    def __repr__(self) -> str:
        return f"<Namespace '{self.id}'>"

    def __hash__(self) -> int:
        return hash(self.id)

    def __lt__(self, other: Any) -> bool:
        if other is None:
            return False
        if isinstance(other, Namespace):
            return self.id < other.id
        return NotImplemented

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, Namespace) and self.id == other.id

    def key(self) -> str:
        return str(self.id)
