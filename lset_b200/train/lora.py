"""LoRA and QLoRA adapters.

``LoRALinear`` wraps a frozen linear layer: ``y = base(x) + lora_B(lora_A(dropout(x))) * alpha / r``
with ``lora_A`` Kaiming-uniform(a=sqrt(5)) and ``lora_B`` zero, so training starts at the base
model. State-dict keys under a wrapped layer are ``base_linear.weight``, ``lora_A.weight``,
``lora_B.weight`` as in the reference (lset/train/lora.py:24-170). For bf16 CUDA tensors the
rank-r update is folded into the base GEMM (``ops.gemm.lora_linear``: the k-blocks of
``(s·x·Aᵀ, B)`` are appended to the contraction of ``(x, W)``), forward and input-gradient alike;
the base weight gets no weight-gradient GEMM because it does not require grad. Quantised bases,
dropout in training mode and tensor-parallel wrappers use the three-product composition.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Iterable, Optional

import torch
import torch.nn as nn

from ..models.layers import Linear

DEFAULT_LORA_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
QWEN3_LORA_TARGETS = DEFAULT_LORA_TARGETS


class LoRALinear(nn.Module):
    def __init__(self, base_linear: nn.Linear, r: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        self.base_linear = base_linear
        for p in self.base_linear.parameters():
            p.requires_grad_(False)
        self.r, self.alpha = r, alpha
        self.scale = alpha / r
        w = base_linear.weight
        # NF4-quantised bases keep their logical shape in in_features / out_features
        self.in_features = getattr(base_linear, "in_features", w.shape[-1])
        self.out_features = getattr(base_linear, "out_features", w.shape[0])
        dtype = w.dtype if w.is_floating_point() else torch.bfloat16
        self.lora_A = Linear(self.in_features, r, bias=False, device=w.device, dtype=dtype)
        self.lora_B = Linear(r, self.out_features, bias=False, device=w.device, dtype=dtype)
        nn.init.kaiming_uniform_(self.lora_A.weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B.weight)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    @property
    def weight(self):
        return self.base_linear.weight

    @property
    def bias(self):
        return self.base_linear.bias

    def _fusable(self, x) -> bool:
        """One-GEMM path: plain bf16 base on the GPU, no dropout mask to apply, no tensor-parallel
        wrappers around the three linears, rank a multiple of 8."""
        b = self.base_linear
        return (type(b) is Linear and x.is_cuda and x.dtype == torch.bfloat16
                and b.weight.dtype == torch.bfloat16 and self.r % 8 == 0
                and (isinstance(self.dropout, nn.Identity) or not self.training)
                and not any(hasattr(m, "_tp_kind") for m in (b, self.lora_A, self.lora_B)))

    def forward(self, x):
        if self._fusable(x):
            from ..ops.gemm import lora_linear

            return lora_linear(x, self.base_linear.weight, self.lora_A.weight, self.lora_B.weight,
                               self.base_linear.bias, self.scale)
        return self.base_linear(x) + self.lora_B(self.lora_A(self.dropout(x))) * self.scale

    def merged_weight(self) -> torch.Tensor:
        """``W + scale * B @ A`` (for export or evaluation without the adapter modules)."""
        base = self.base_linear.weight
        if hasattr(self.base_linear, "dequantized_weight"):
            base = self.base_linear.dequantized_weight()
        return base.float() + self.scale * (self.lora_B.weight.float() @ self.lora_A.weight.float())


def _wrap_targets(model: nn.Module, targets: Iterable[str], r, alpha, dropout) -> int:
    wanted, n = set(targets), 0
    for fqn, mod in list(model.named_modules()):
        if not isinstance(mod, nn.Linear) or fqn.rsplit(".", 1)[-1] not in wanted:
            continue
        parent = model.get_submodule(fqn.rsplit(".", 1)[0]) if "." in fqn else model
        setattr(parent, fqn.rsplit(".", 1)[-1], LoRALinear(mod, r=r, alpha=alpha, dropout=dropout))
        n += 1
    leaves = {fqn.rsplit(".", 1)[-1] for fqn, _ in model.named_modules()}
    missing = sorted(t for t in wanted if t not in leaves)
    if missing:
        fused = sorted(leaves & {"qkv_proj", "gate_up_proj"})
        hint = (f"; this model has fused projections {fused}: name them as targets or load it with "
                f"model.fused_projections: false") if fused else ""
        print(f"[lset_b200] LoRA targets without a matching layer: {missing}{hint}")
    return n


def apply_lora(model: nn.Module, r: int = 8, alpha: float = 16.0,
               target_modules: Optional[Iterable[str]] = None, dropout: float = 0.0) -> nn.Module:
    """Freeze every parameter, then wrap each ``nn.Linear`` whose leaf name is a target."""
    for p in model.parameters():
        p.requires_grad_(False)
    _wrap_targets(model, target_modules or DEFAULT_LORA_TARGETS, r, alpha, dropout)
    return model


def apply_qlora(model: nn.Module, r: int = 8, alpha: float = 16.0,
                target_modules: Optional[Iterable[str]] = None, dropout: float = 0.0,
                block_size: int = 64, scaler_block_size: int = 256) -> nn.Module:
    """NF4-quantise the target linears (frozen), then add LoRA adapters on top."""
    from .quantization.nf4 import quantize_linear_nf4

    targets = set(target_modules or DEFAULT_LORA_TARGETS)
    for p in model.parameters():
        p.requires_grad_(False)
    for fqn, mod in list(model.named_modules()):
        if isinstance(mod, nn.Linear) and fqn.rsplit(".", 1)[-1] in targets:
            parent = model.get_submodule(fqn.rsplit(".", 1)[0]) if "." in fqn else model
            setattr(parent, fqn.rsplit(".", 1)[-1],
                    quantize_linear_nf4(mod, block_size=block_size, scaler_block_size=scaler_block_size))
    # NF4 layers are nn.Linear subclasses, so the same wrapping pass picks them up
    _wrap_targets(model, targets, r, alpha, dropout)
    return model


def get_lora_params(model: nn.Module):
    return [p for p in model.parameters() if p.requires_grad]


def save_lora_weights(model: nn.Module, path: str) -> None:
    state = OrderedDict((n, p.detach().cpu().clone()) for n, p in model.named_parameters()
                        if p.requires_grad and ("lora_A" in n or "lora_B" in n))
    torch.save(state, path)


def load_lora_weights(model: nn.Module, path: str) -> None:
    state = torch.load(path, map_location="cpu", weights_only=True)
    missing_ok = model.load_state_dict(state, strict=False)
    unexpected = list(missing_ok.unexpected_keys)
    if unexpected:
        raise KeyError(f"adapter file has keys the model lacks: {unexpected[:5]}")
