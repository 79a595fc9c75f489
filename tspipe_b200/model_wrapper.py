"""Pytree-valued stage interfaces (`tspipe/model_wrapper.py:7-27`).

A stage wrapped in :class:`TSPipeModelWrapper` may take and return arbitrary pytrees
(lists, tuples, dicts, ``None``/scalars as leaves).  The runtime flattens the tree,
moves the tensor leaves over the stage link one by one and rebuilds the tree on the
other side; leaves that require grad get a gradient edge back (the reference finds
those paths with `tspipe/utils.py:294-325`)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Tuple, Union

import torch


@dataclass
class TSPipeModelOutput:
    data: Any
    lst_require_grad_tensor_path: Optional[List[Tuple]] = None


class TSPipeModelWrapper(torch.nn.Module):
    def __init__(self, model: torch.nn.Module):
        super().__init__()
        self.model = model

    def forward(self, input) -> Union[TSPipeModelOutput, torch.Tensor]:
        out = self.model(input.data if isinstance(input, TSPipeModelOutput) else input)
        if isinstance(out, torch.Tensor):
            return out
        return TSPipeModelOutput(data=out, lst_require_grad_tensor_path=None)
