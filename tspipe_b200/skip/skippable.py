"""Skip connections that may cross pipeline stages.

Public surface of the reference's (vendored, not importable) copy of torchgpipe's skip API
(`tspipe/skip/skippable.py:213-289` ``@skippable``, `:292-332` ``stash`` / ``pop``, `:335-416`
``verify_skippables``; `tspipe/skip/layout.py:11-83`; `tspipe/skip/tracker.py`):

    @skippable(stash=["skip"])
    class Stash(nn.Module):
        def forward(self, x):
            yield stash("skip", x)
            return f(x)

    @skippable(pop=["skip"])
    class Pop(nn.Module):
        def forward(self, x):
            skip = yield pop("skip")
            return g(x) + skip

Mechanism here (instead of portals and phony autograd edges, `tspipe/skip/portal.py`): a partition
that contains skippable layers runs inside a :class:`SkipScope`.  Tensors stashed but not popped by
the end of the partition leave the stage as extra leaves of its output pytree
(:data:`MAIN_KEY` / :data:`SKIPS_KEY`), travel over the ordinary stage link - so they are prefetched,
overlapped and get their gradient sent back exactly like the activation - and are re-seeded into the
scope of the next stage, hop by hop until the partition that pops them.  Within one stage a skip is a
plain tensor reference, i.e. normal autograd.
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from typing import Any, Callable, Dict, Generator, Iterable, List, Optional, Sequence, Set, Tuple, Type, TypeVar

from torch import Tensor, nn

from .namespace import Namespace

__all__ = ["skippable", "stash", "pop", "verify_skippables", "Skippable", "SkipSequential", "MAIN_KEY", "SKIPS_KEY"]

MAIN_KEY = "__tspipe_main__"
SKIPS_KEY = "__tspipe_skips__"
T = TypeVar("T", bound=nn.Module)


class stash:
    """``yield stash(name, tensor)`` inside a skippable ``forward``."""
    __slots__ = ("name", "tensor")

    def __init__(self, name: str, tensor: Optional[Tensor]) -> None:
        self.name, self.tensor = name, tensor


class pop:
    """``tensor = yield pop(name)`` inside a skippable ``forward``."""
    __slots__ = ("name",)

    def __init__(self, name: str) -> None:
        self.name = name


def _key(ns: Optional[Namespace], name: str) -> str:
    return f"{ns.key() if ns is not None else ''}/{name}"


class SkipScope:
    """Skip tensors alive during one forward call of one partition (thread-local, re-entrant)."""
    _tls = threading.local()

    def __init__(self, seed: Optional[Dict[str, Tensor]] = None):
        self.tensors: Dict[str, Optional[Tensor]] = dict(seed or {})

    def __enter__(self) -> "SkipScope":
        stack = getattr(self._tls, "stack", None)
        if stack is None:
            stack = self._tls.stack = []
        stack.append(self)
        return self

    def __exit__(self, *exc) -> None:
        self._tls.stack.pop()

    @classmethod
    def current(cls) -> "SkipScope":
        stack = getattr(cls._tls, "stack", None)
        if not stack:
            raise RuntimeError("a skippable layer ran outside a SkipSequential / SkipScope")
        return stack[-1]


class Skippable(nn.Module):
    """Wrapper produced by :func:`skippable` (`tspipe/skip/skippable.py:27-209`)."""
    module_cls: Type[nn.Module]
    stashable_names: Set[str]
    poppable_names: Set[str]

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__()
        self.module = self.module_cls(*args, **kwargs)
        self.namespaces: Dict[str, Namespace] = {}

    def __repr__(self) -> str:
        return f"@skippable({self.module})"

    def namespaced(self, name: str) -> Tuple[Optional[Namespace], str]:
        return self.namespaces.get(name), name

    def stashable(self) -> Iterable[Tuple[Optional[Namespace], str]]:
        for name in self.stashable_names:
            yield self.namespaced(name)

    def poppable(self) -> Iterable[Tuple[Optional[Namespace], str]]:
        for name in self.poppable_names:
            yield self.namespaced(name)

    def isolate(self: T, ns: Namespace, *, only: Optional[Iterable[str]] = None) -> T:
        names = set(only) if only is not None else self.stashable_names | self.poppable_names
        for name in names:
            self.namespaces[name] = ns
        return self

    def forward(self, input: Any) -> Any:  # type: ignore[override]
        scope = SkipScope.current()
        gen = self.module(input)
        if not isinstance(gen, Generator):
            return gen                      # a forward without any yield
        stashed, popped = set(), set()
        try:
            op = next(gen)
            while True:
                if isinstance(op, stash):
                    if op.name not in self.stashable_names:
                        raise RuntimeError(f"'{op.name}' has not been declared as stashable")
                    scope.tensors[_key(*self.namespaced(op.name))] = op.tensor
                    stashed.add(op.name)
                    op = gen.send(None)
                elif isinstance(op, pop):
                    if op.name not in self.poppable_names:
                        raise RuntimeError(f"'{op.name}' has not been declared as poppable")
                    k = _key(*self.namespaced(op.name))
                    if k not in scope.tensors:
                        raise RuntimeError(f"'{op.name}' is popped before any layer stashed it")
                    popped.add(op.name)
                    op = gen.send(scope.tensors.pop(k))
                else:
                    raise TypeError(f"{op!r} is not a stash or pop")
        except StopIteration as stop:
            output = stop.value
        missing = (self.stashable_names - stashed) | (self.poppable_names - popped)
        if missing:
            raise RuntimeError(f"{', '.join(sorted(missing))} declared but not stashed/popped by {self.module}")
        return output


def skippable(stash: Iterable[str] = (), pop: Iterable[str] = ()) -> Callable[[Type[nn.Module]], Type[Skippable]]:
    """Class decorator: declare which skip names the module's generator-style ``forward`` stashes and pops."""
    stashable, poppable = frozenset(stash), frozenset(pop)

    def extend(module_cls: Type[nn.Module]) -> Type[Skippable]:
        name = module_cls.__name__
        return type(name, (Skippable,), {"module_cls": module_cls, "stashable_names": set(stashable),
                                         "poppable_names": set(poppable), "__module__": module_cls.__module__,
                                         "__qualname__": getattr(module_cls, "__qualname__", name)})
    return extend


def _skippables(module: nn.Module) -> List[Tuple[str, Skippable]]:
    return [(n, m) for n, m in module.named_children() if isinstance(m, Skippable)]


def verify_skippables(module: nn.Sequential) -> None:
    """Every stashed name is popped exactly once, later, and nothing is popped that was not stashed
    (`tspipe/skip/skippable.py:335-416`).  Raises ``TypeError`` listing every violation."""
    stashed: Set[Tuple[Optional[Namespace], str]] = set()
    popped: Set[Tuple[Optional[Namespace], str]] = set()
    msgs: List[str] = []
    for layer_name, layer in module.named_children():
        if not isinstance(layer, Skippable):
            continue
        for name in layer.stashable_names & layer.poppable_names:
            msgs.append(f"'{layer_name}' declared '{name}' both as stashable and as poppable")
        for ns, name in layer.stashable():
            if name in layer.poppable_names:
                continue
            if (ns, name) in stashed:
                msgs.append(f"'{layer_name}' redeclared '{name}' as stashable but not isolated by namespace")
            stashed.add((ns, name))
        for ns, name in layer.poppable():
            if name in layer.stashable_names:
                continue
            if (ns, name) in popped:
                msgs.append(f"'{layer_name}' redeclared '{name}' as poppable but not isolated by namespace")
            elif (ns, name) not in stashed:
                msgs.append(f"'{layer_name}' declared '{name}' as poppable but it was not stashed")
            popped.add((ns, name))
    for ns, name in stashed - popped:
        msgs.append(f"no module declared '{name}' as poppable but stashed")
    if msgs:
        raise TypeError("one or more pairs of stash and pop do not match:\n\n" + "".join(f"* {m}\n" for m in msgs))


class SkipSequential(nn.Sequential):
    """A partition with skippable layers.  Input and output may carry skip tensors from / for other
    stages as ``{MAIN_KEY: activation, SKIPS_KEY: {key: tensor}}``."""

    def forward(self, input: Any) -> Any:  # type: ignore[override]
        seed: Dict[str, Tensor] = {}
        if isinstance(input, dict) and MAIN_KEY in input:
            seed = dict(input.get(SKIPS_KEY, {}))
            input = input[MAIN_KEY]
        with SkipScope(seed) as scope:
            for layer in self:
                input = layer(input)
            left = {k: v for k, v in scope.tensors.items() if v is not None}
        if left:
            return {MAIN_KEY: input, SKIPS_KEY: left}
        return input


def wrap_partitions(partitions: Sequence[nn.Sequential]) -> List[nn.Sequential]:
    """Turn partitions into :class:`SkipSequential` when the model uses skippable layers anywhere."""
    if not any(isinstance(m, Skippable) for p in partitions for m in p.children()):
        return list(partitions)
    return [SkipSequential(OrderedDict(p.named_children())) if not isinstance(p, SkipSequential) else p for p in partitions]
