"""Learning-rate / momentum schedules used by the training entry points
(`benchmarks/byol/trainer.py:282-295`, `benchmarks/moco-v3/main.py:534-548`)."""
from __future__ import annotations

import math


def cosine_lr(epoch: float, total_epochs: int, base_lr: float, warmup_epochs: int = 10) -> float:
    """Linear warm-up then half-cosine decay."""
    if epoch < warmup_epochs:
        return base_lr * epoch / max(warmup_epochs, 1)
    return base_lr * 0.5 * (1.0 + math.cos(math.pi * (epoch - warmup_epochs) / max(total_epochs - warmup_epochs, 1)))


def cosine_momentum(epoch: float, total_epochs: int, base_m: float) -> float:
    """Momentum rising from ``base_m`` to 1 along a half cosine."""
    return 1.0 - 0.5 * (1.0 + math.cos(math.pi * epoch / max(total_epochs, 1))) * (1.0 - base_m)


def linear_warmup_decay(step: int, total_steps: int, base_lr: float, warmup_steps: int) -> float:
    """Linear warm-up / linear decay (`benchmarks/distilbert/distiller.py:150-157`)."""
    if step < warmup_steps:
        return base_lr * step / max(warmup_steps, 1)
    return base_lr * max(0.0, (total_steps - step) / max(total_steps - warmup_steps, 1))
