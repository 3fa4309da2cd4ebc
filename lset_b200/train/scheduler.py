"""Learning-rate schedules: linear warm-up, then constant / cosine / linear / warmup-stable-decay
(curves of lset/train/scheduler.py:8-38). Works with any optimizer object that exposes
``param_groups`` (torch optimizers and ``ShardedAdamW``)."""
from __future__ import annotations

import math


def lr_factor(step: int, kind: str, warmup_steps: int, total_steps: int, stable_ratio: float = 0.7):
    """Multiplier of the base learning rate at ``step`` (0-based count of completed updates)."""
    if warmup_steps > 0 and step < warmup_steps:
        return step / warmup_steps
    span = max(1, total_steps - warmup_steps)
    progress = min(1.0, (step - warmup_steps) / span)
    if kind == "constant":
        return 1.0
    if kind == "cosine":
        return 0.5 * (1.0 + math.cos(math.pi * progress))
    if kind == "linear":
        return max(0.0, 1.0 - progress)
    if kind == "wsd":
        if progress < stable_ratio:
            return 1.0
        tail = (progress - stable_ratio) / max(1e-12, 1.0 - stable_ratio)
        return 0.5 * (1.0 + math.cos(math.pi * min(1.0, tail)))
    raise ValueError(f"Unknown scheduler: {kind}")


class LRSchedule:
    def __init__(self, optimizer, kind: str = "cosine", warmup_steps: int = 0,
                 total_steps: int = 1000, stable_ratio: float = 0.7):
        lr_factor(0, kind, warmup_steps, total_steps)  # validates ``kind``
        self.optimizer = optimizer
        self.kind, self.warmup_steps, self.total_steps = kind, warmup_steps, total_steps
        self.stable_ratio = stable_ratio
        self.base_lrs = [g.setdefault("initial_lr", g["lr"]) for g in optimizer.param_groups]
        self.last_step = 0
        self._apply()

    def _apply(self):
        f = lr_factor(self.last_step, self.kind, self.warmup_steps, self.total_steps,
                      self.stable_ratio)
        for g, base in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = base * f

    def step(self):
        self.last_step += 1
        self._apply()

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"last_step": self.last_step, "base_lrs": list(self.base_lrs)}

    def load_state_dict(self, sd):
        self.last_step = int(sd["last_step"])
        self.base_lrs = list(sd.get("base_lrs", self.base_lrs))
        self._apply()


def build_scheduler(optimizer, scheduler_type: str = "cosine", warmup_steps: int = 0,
                    total_steps: int = 1000) -> LRSchedule:
    return LRSchedule(optimizer, scheduler_type, warmup_steps, total_steps)
