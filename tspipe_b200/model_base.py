"""Base class for models that can turn themselves into a cut-able ``nn.Sequential``
(`tspipe/model_base.py:7-36`)."""
from __future__ import annotations

from typing import Iterable

import torch
from torch import nn


class SequentialableModel(nn.Module):
    def to_sequential(self) -> nn.Sequential:
        raise NotImplementedError(f"to_sequential is not implemented for {self.__class__}.")

    def test_sequential_validity(self, test_tensor_size: Iterable[int], rtol: float = 1e-5, atol: float = 1e-6) -> bool:
        """Evaluation-mode outputs of the original module and of its sequential form agree."""
        x = torch.rand(tuple(test_tensor_size))
        seq = self.to_sequential()
        was_training = self.training
        with torch.no_grad():
            self.eval()
            seq.eval()
            ok = torch.allclose(self(x), seq(x), rtol=rtol, atol=atol)
        self.train(was_training)
        return bool(ok)


class FlattenWrapper(nn.Module):
    def __init__(self, *args, **kwargs):
        super().__init__()
        self._args, self._kwargs = args, kwargs

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x.flatten(*self._args, **self._kwargs)
