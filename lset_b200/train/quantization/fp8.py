"""FP8 training (cf. lset/train/quantization/fp8.py:11-75, which delegates to torchao).

``apply_fp8_training(model, recipe)`` swaps every eligible linear layer (both dims multiples of 16)
for ``Float8Linear``: activations, weights and output gradients are quantised to float8 with
``tensorwise`` or ``rowwise`` (``rowwise_with_gw_hp``: weight gradient kept in high precision)
dynamic scaling — e4m3 for forward operands, e5m2 for gradients — and the products run on the bf16
tcgen05 GEMM after dequantisation. This reproduces FP8 *numerics* (what matters for convergence
studies and for checkpoints) but not yet FP8 *throughput*: a kind::f8f6f4 tensor-core kernel is
not part of this library, and that is stated here rather than hidden. ``get_fp8_tp_plan`` mirrors
the reference's plan helper.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn

from ...ops.gemm import linear as gemm_linear

RECIPES = ("tensorwise", "rowwise", "rowwise_with_gw_hp")
E4M3_MAX, E5M2_MAX = 448.0, 57344.0


def fake_quant_fp8(x: torch.Tensor, rowwise: bool, dtype=torch.float8_e4m3fn) -> torch.Tensor:
    """Quantise to float8 with a dynamic scale (per tensor or per row) and dequantise back."""
    fmax = E4M3_MAX if dtype == torch.float8_e4m3fn else E5M2_MAX
    xf = x.float()
    amax = xf.abs().amax(dim=-1, keepdim=True) if rowwise else xf.abs().amax()
    scale = fmax / amax.clamp(min=1e-12)
    return ((xf * scale).to(dtype).float() / scale).to(x.dtype)


class _Fp8Matmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, rowwise, hp_wgrad):
        ctx.save_for_backward(x, w)
        ctx.rowwise, ctx.hp_wgrad = rowwise, hp_wgrad
        return gemm_linear(fake_quant_fp8(x, rowwise), fake_quant_fp8(w, rowwise))

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        rw = ctx.rowwise
        dyq = fake_quant_fp8(dy, rw, torch.float8_e5m2)
        dy2, x2 = dyq.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        dx = (dy2 @ fake_quant_fp8(w, rw)).view_as(x) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            a = dy.reshape(-1, dy.shape[-1]) if ctx.hp_wgrad else dy2
            b = x2 if ctx.hp_wgrad else fake_quant_fp8(x2, rw)
            dw = (a.float().t() @ b.float()).to(w.dtype)
        return dx, dw, None, None


class Float8Linear(nn.Linear):
    recipe = "rowwise"

    def forward(self, x):
        rw = self.recipe != "tensorwise"
        y = _Fp8Matmul.apply(x, self.weight, rw, self.recipe == "rowwise_with_gw_hp")
        return y + self.bias if self.bias is not None else y


def _eligible(m: nn.Linear) -> bool:
    return m.in_features % 16 == 0 and m.out_features % 16 == 0


def apply_fp8_training(model: nn.Module, recipe: str = "rowwise") -> nn.Module:
    if recipe not in RECIPES:
        raise ValueError(f"Unknown FP8 recipe {recipe!r}; choose from {RECIPES}")
    for mod in model.modules():
        if isinstance(mod, nn.Linear) and _eligible(mod) and type(mod).__name__ in ("Linear",):
            mod.__class__ = Float8Linear
            mod.recipe = recipe
    return model


def get_fp8_tp_plan(fused_projections: bool = False) -> Dict[str, str]:
    from ...models.parallel_plan import decoder_tp_plan

    return decoder_tp_plan(None, fused_projections=fused_projections)
