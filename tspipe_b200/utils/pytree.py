"""Pytree helpers for stage inputs/outputs and user batches.

Same jobs as the reference's traversal helpers (`tspipe/utils.py:179-325`:
``traverse_tensor_map``, ``generic_object_scatter/gather``,
``find_path_tensor_requires_grad``), built on ``torch.utils._pytree``."""
from __future__ import annotations

from typing import Any, Callable, List, Sequence, Tuple

import torch
import torch.utils._pytree as pytree

from ..model_wrapper import TSPipeModelOutput


def unwrap(obj: Any) -> Any:
    return obj.data if isinstance(obj, TSPipeModelOutput) else obj


def flatten(obj: Any) -> Tuple[List[Any], Any, bool]:
    """(leaves, treespec, was_wrapped)."""
    wrapped = isinstance(obj, TSPipeModelOutput)
    leaves, spec = pytree.tree_flatten(unwrap(obj))
    return leaves, spec, wrapped


def unflatten(leaves: Sequence[Any], spec: Any, wrapped: bool = False) -> Any:
    obj = pytree.tree_unflatten(list(leaves), spec)
    return TSPipeModelOutput(obj, None) if wrapped else obj


def tree_map_tensors(fn: Callable[[torch.Tensor], Any], obj: Any) -> Any:
    wrapped = isinstance(obj, TSPipeModelOutput)
    out = pytree.tree_map(lambda x: fn(x) if isinstance(x, torch.Tensor) else x, unwrap(obj))
    return TSPipeModelOutput(out, None) if wrapped else out


def tree_map_tensors_multi(fn: Callable[..., Any], first: Any, *rest: Any) -> Any:
    """``fn(leaf_of_first, leaf_of_rest_0, ...)`` on the tensor leaves of equally structured pytrees; other
    leaves are taken from ``first``."""
    leaves, spec, wrapped = flatten(first)
    others = [flatten(r)[0] for r in rest]
    out = [fn(l, *[o[i] for o in others]) if isinstance(l, torch.Tensor) else l for i, l in enumerate(leaves)]
    return unflatten(out, spec, wrapped)


def tensors_of(obj: Any) -> List[torch.Tensor]:
    return [x for x in pytree.tree_leaves(unwrap(obj)) if isinstance(x, torch.Tensor)]


def generic_scatter(obj: Any, chunks: int) -> List[Any]:
    """Chunk every tensor leaf along dim 0; non-tensor leaves are replicated."""
    leaves, spec, wrapped = flatten(obj)
    pieces: List[List[Any]] = [[] for _ in range(chunks)]
    for leaf in leaves:
        if isinstance(leaf, torch.Tensor) and leaf.dim() > 0:
            parts = leaf.chunk(chunks)
            if len(parts) != chunks:
                raise ValueError(f"cannot split a leading dimension of {leaf.shape[0]} into {chunks} chunks")
            for i in range(chunks):
                pieces[i].append(parts[i])
        else:
            for i in range(chunks):
                pieces[i].append(leaf)
    return [unflatten(p, spec, wrapped) for p in pieces]


def generic_gather(objs: Sequence[Any]) -> Any:
    """Inverse of :func:`generic_scatter` (concatenate tensor leaves along dim 0)."""
    flat = [flatten(o) for o in objs]
    spec, wrapped = flat[0][1], flat[0][2]
    out = []
    for i, leaf in enumerate(flat[0][0]):
        if isinstance(leaf, torch.Tensor) and leaf.dim() > 0:
            out.append(torch.cat([f[0][i] for f in flat]) if len(flat) > 1 else leaf)
        else:
            out.append(leaf)
    return unflatten(out, spec, wrapped)


def leading_size(obj: Any) -> int:
    for t in tensors_of(obj):
        if t.dim() > 0:
            return t.shape[0]
    raise ValueError("no tensor with a batch dimension in the object")
