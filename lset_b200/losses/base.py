"""Learnable or fixed logit scale (inverse temperature), cf. lset/losses/base.py:11-36."""
from __future__ import annotations

import math

import torch
import torch.nn as nn


class LogitScale(nn.Module):
    """``scale = exp(log_scale)`` clamped to ``max_scale``; a parameter when ``learnable``."""

    def __init__(self, init_scale: float = 50.0, learnable: bool = False, max_scale: float = 100.0):
        super().__init__()
        value = torch.tensor(math.log(init_scale), dtype=torch.float32)
        if learnable:
            self.log_scale = nn.Parameter(value)
        else:
            self.register_buffer("log_scale", value)
        self.max_scale = max_scale
        self.learnable = learnable

    @classmethod
    def from_temperature(cls, temperature: float, learnable: bool = False,
                         max_scale: float = 100.0) -> "LogitScale":
        return cls(1.0 / temperature, learnable, max(max_scale, 1.0 / temperature))

    def forward(self) -> torch.Tensor:
        return self.log_scale.exp().clamp(max=self.max_scale)
