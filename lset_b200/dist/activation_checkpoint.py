"""Activation checkpointing of transformer blocks.

``full``: the bottom ``ratio`` fraction of blocks recompute their whole forward in backward.
``selective``: the same blocks are checkpointed, but the outputs of the expensive ops — the GEMMs
and attention of this framework — are kept and handed back during the recompute; norms, RoPE,
activations and pooling are recomputed. This is the reference's policy (MUST_SAVE for mm / addmm /
bmm / SDPA, everything else recomputed; lset/distributed/parallel.py:81-126) expressed for custom
ops. Blocks are patched in place (their ``forward`` is wrapped), so parameter names do not change.
"""
from __future__ import annotations

import functools

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..ops import _ac


def _checkpointed_forward(block: nn.Module, mode: str):
    inner = block.forward

    @functools.wraps(inner)
    def forward(*args, **kwargs):
        if not torch.is_grad_enabled():
            return inner(*args, **kwargs)
        if mode == "full":
            return checkpoint(inner, *args, use_reentrant=False, **kwargs)
        saved = _ac.SavedOutputs()
        return checkpoint(inner, *args, use_reentrant=False,
                          context_fn=lambda: (_ac.recording(saved), _ac.replaying(saved)), **kwargs)

    forward._lset_ac_mode = mode
    return forward


def apply_activation_checkpointing(model: nn.Module, mode: str = "selective", ratio: float = 1.0) -> nn.Module:
    """Checkpoint the bottom ``ratio * L`` blocks of ``model.layers``."""
    if mode not in ("selective", "full"):
        raise ValueError(f"Unknown activation checkpoint mode: {mode}")
    layers = getattr(model, "layers", None)
    if layers is None:
        return model
    n = int(round(max(0.0, min(1.0, ratio)) * len(layers)))
    for i in range(n):
        if not hasattr(layers[i].forward, "_lset_ac_mode"):
            layers[i].forward = _checkpointed_forward(layers[i], mode)
    return model


def checkpointed_layers(model: nn.Module):
    return [i for i, l in enumerate(getattr(model, "layers", [])) if hasattr(l.forward, "_lset_ac_mode")]


_apply_ac = apply_activation_checkpointing
