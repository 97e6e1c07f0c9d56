"""Learning-rate schedule with warm-up and constant / linear / cosine decay, checkpointable.
Same behaviour as the reference AnnealingLR (runtime/megatron/learning_rates.py:22-164)."""
from __future__ import annotations

import math


class LRSchedule:
    def __init__(self, max_lr: float, min_lr: float = 0.0, warmup_steps: int = 0, decay_steps: int = 1,
                 style: str = "cosine"):
        assert style in ("constant", "linear", "cosine")
        assert 0.0 <= min_lr <= max_lr and decay_steps > 0 and warmup_steps < decay_steps or style == "constant"
        self.max_lr, self.min_lr = float(max_lr), float(min_lr)
        self.warmup_steps, self.decay_steps, self.style = warmup_steps, decay_steps, style
        self.num_steps = 0

    def get_lr(self) -> float:
        n = self.num_steps
        if self.warmup_steps > 0 and n <= self.warmup_steps:
            return self.max_lr * n / self.warmup_steps
        if self.style == "constant":
            return self.max_lr
        if n > self.decay_steps:
            return self.min_lr
        ratio = (n - self.warmup_steps) / (self.decay_steps - self.warmup_steps)
        delta = self.max_lr - self.min_lr
        coeff = (1.0 - ratio) if self.style == "linear" else 0.5 * (math.cos(math.pi * ratio) + 1.0)
        return self.min_lr + coeff * delta

    def step(self, increment: int = 1) -> float:
        self.num_steps += increment
        return self.get_lr()

    def state_dict(self) -> dict:
        return {"max_lr": self.max_lr, "min_lr": self.min_lr, "warmup_steps": self.warmup_steps,
                "decay_steps": self.decay_steps, "decay_style": self.style, "num_steps": self.num_steps}

    def load_state_dict(self, sd: dict) -> None:
        self.max_lr, self.min_lr = sd["max_lr"], sd["min_lr"]
        self.warmup_steps, self.decay_steps = sd["warmup_steps"], sd["decay_steps"]
        self.style, self.num_steps = sd["decay_style"], sd["num_steps"]
