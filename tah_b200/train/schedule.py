"""Learning-rate schedules used by the recipes: linear warm-up then cosine decay to
``min_lr_rate * lr`` (HuggingFace's ``cosine_with_min_lr``), plus plain linear / constant."""
from __future__ import annotations

import math


def lr_factor(step: int, total_steps: int, warmup_steps: int, kind: str = "cosine_with_min_lr",
              min_lr_rate: float = 0.0, num_cycles: float = 0.5) -> float:
    if warmup_steps > 0 and step < warmup_steps:
        return step / max(1, warmup_steps)
    if kind in ("constant", "constant_with_warmup"):
        return 1.0
    progress = (step - warmup_steps) / max(1, total_steps - warmup_steps)
    progress = min(max(progress, 0.0), 1.0)
    if kind == "linear":
        return max(0.0, 1.0 - progress)
    cos = 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * progress))
    if kind == "cosine":
        return max(0.0, cos)
    return cos * (1.0 - min_lr_rate) + min_lr_rate          # cosine_with_min_lr
