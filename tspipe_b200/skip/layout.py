"""Static view of which skip tensors cross which partitions (`tspipe/skip/layout.py:11-83`)."""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from torch import nn

from .namespace import Namespace
from .skippable import Skippable


class SkipLayout:
    def __init__(self, num_partitions: int, skip_routes: Dict[Tuple[Optional[Namespace], str], Tuple[int, int]]):
        self.num_partitions = num_partitions
        self.skip_routes = skip_routes
        self.by_partition: List[List[Tuple[int, Optional[Namespace], str]]] = [[] for _ in range(num_partitions)]
        for (ns, name), (prev_j, next_j) in skip_routes.items():
            self.by_partition[next_j].append((prev_j, ns, name))
        for x in self.by_partition:
            x.sort(key=lambda t: (t[0], t[2]))

    def copy_policy(self, next_j: int) -> Iterable[Tuple[int, Optional[Namespace], str]]:
        """Skips that arrive at partition ``next_j`` from another partition: ``(source, ns, name)``."""
        for prev_j, ns, name in self.by_partition[next_j]:
            if prev_j != next_j:
                yield prev_j, ns, name

    def requires_copy(self, ns: Optional[Namespace], name: str) -> bool:
        prev_j, next_j = self.skip_routes.get((ns, name), (-1, -1))
        return prev_j != next_j

    def hops(self) -> Dict[int, List[Tuple[Optional[Namespace], str]]]:
        """For each stage boundary ``j`` (between partition ``j`` and ``j+1``) the skips that ride over it."""
        out: Dict[int, List[Tuple[Optional[Namespace], str]]] = {j: [] for j in range(self.num_partitions - 1)}
        for key, (a, b) in self.skip_routes.items():
            for j in range(a, b):
                out[j].append(key)
        return out


def inspect_skip_layout(partitions: Sequence[nn.Sequential]) -> SkipLayout:
    routes: Dict[Tuple[Optional[Namespace], str], Tuple[int, int]] = {}
    stashed_at: Dict[Tuple[Optional[Namespace], str], int] = {}
    for j, partition in enumerate(partitions):
        for layer in partition.children():
            if not isinstance(layer, Skippable):
                continue
            for ns, name in layer.stashable():
                stashed_at[(ns, name)] = j
            for ns, name in layer.poppable():
                routes[(ns, name)] = (stashed_at.pop((ns, name)), j)
    return SkipLayout(len(partitions), routes)
