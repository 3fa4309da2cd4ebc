"""FP8 training (cf. lset/train/quantization/fp8.py:11-75, which delegates to torchao).

``apply_fp8_training(model, recipe)`` swaps every eligible linear layer (both dims multiples of 16)
for ``Float8Linear``. Its three products run on the 8-bit tensor-core GEMM (``ops/fp8.py``:
``tcgen05.mma kind::f8f6f4``, fp32 accumulation, dequantisation in the epilogue) with dynamic
scaling — e4m3 for activations and weights, e5m2 for output gradients:

``tensorwise``
    one scale per tensor. Each tensor is cast once; the cast kernel emits the row-major and the
    transposed copy together, the backward pass keeps only the 8-bit copies of ``x`` and ``w``.
``rowwise``
    one scale per slice *along the contraction* of each product, so every product re-casts its
    operands: fprop scales ``x`` per token and ``w`` per output feature, dgrad scales ``dy`` per
    token and ``w`` per input feature, wgrad scales ``dy`` per output feature and ``x`` per input
    feature (both over the tokens).
``rowwise_with_gw_hp``
    as ``rowwise`` but the weight gradient is computed from the bf16 tensors.

Weight gradients go straight into the fp32 accumulator of the sharding runtime when the weight has
one. On the CPU the same quantise → multiply → rescale arithmetic runs in plain PyTorch.
``get_fp8_tp_plan`` mirrors the reference's plan helper.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn

from ...ops import fp8 as f8
from ...ops._grads import main_grad_of
from ...ops.gemm import _accumulate_wgrad, wgrad_splits

RECIPES = ("tensorwise", "rowwise", "rowwise_with_gw_hp")
E4M3_MAX, E5M2_MAX = f8.E4M3_MAX, f8.E5M2_MAX


def fake_quant_fp8(x: torch.Tensor, rowwise: bool, dtype=torch.float8_e4m3fn) -> torch.Tensor:
    """Quantise to float8 with a dynamic scale (per tensor or per row) and dequantise back."""
    fmax = E4M3_MAX if dtype == torch.float8_e4m3fn else E5M2_MAX
    xf = x.float()
    amax = xf.abs().amax(dim=-1, keepdim=True) if rowwise else xf.abs().amax()
    scale = fmax / amax.clamp(min=1e-12)
    return ((xf * scale).to(dtype).float() / scale).to(x.dtype)


def _wgrad(w, a_t: f8.Fp8Tensor, b_t: f8.Fp8Tensor, tokens: int):
    """``dW = dyᵀ · x`` from the transposed 8-bit copies ``a_t [N, T]``, ``b_t [K, T]``."""
    main = main_grad_of(w)
    splits = wgrad_splits(w.shape[0], w.shape[1], tokens) if a_t.data.is_cuda else 1
    if main is not None and a_t.data.is_cuda:
        f8.matmul_fp8(a_t, b_t, out=main, accumulate=True, splits=splits)
        return None
    return f8.matmul_fp8(a_t, b_t, out_dtype=torch.float32, splits=splits).to(w.dtype)


class _Fp8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, rowwise, hp_wgrad):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.rowwise, ctx.hp_wgrad, ctx.has_bias = rowwise, hp_wgrad, bias is not None
        ctx.x_shape, ctx.tokens = x.shape, x2.shape[0]
        ctx.act_dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16
        if rowwise:
            xq, _ = f8.quantize_fp8(x2, f8.PER_ROW)
            wq, _ = f8.quantize_fp8(w, f8.PER_ROW)
            ctx.save_for_backward(x, w)
        else:
            xq, xq_t = f8.quantize_fp8(x2, f8.PER_TENSOR, want_t=True)
            wq, wq_t = f8.quantize_fp8(w, f8.PER_TENSOR, want_t=True)
            # the backward pass needs only the transposed 8-bit copies
            ctx.save_for_backward(xq_t.data, xq_t.inv_scale, wq_t.data, wq_t.inv_scale, w)
        y = f8.matmul_fp8(xq, wq, bias=bias, out_dtype=ctx.act_dtype)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16 and dy2.is_cuda:
            dy2 = dy2.to(torch.bfloat16)
        T = ctx.tokens
        dx = dw = db = None
        if ctx.rowwise:
            x, w = ctx.saved_tensors
            x2 = x.reshape(-1, x.shape[-1])
            if ctx.needs_input_grad[0]:
                dyq, _ = f8.quantize_fp8(dy2, f8.PER_ROW, e5m2=True)
                _, wq_t = f8.quantize_fp8(w, f8.PER_COL, want=False, want_t=True)
                dx = f8.matmul_fp8(dyq, wq_t, out_dtype=ctx.act_dtype).view(ctx.x_shape)
            if ctx.needs_input_grad[1]:
                if ctx.hp_wgrad:
                    dw = _accumulate_wgrad(w, dy2.contiguous(), x2)
                else:
                    _, dyq_t = f8.quantize_fp8(dy2, f8.PER_COL, e5m2=True, want=False, want_t=True)
                    _, xq_t = f8.quantize_fp8(x2, f8.PER_COL, want=False, want_t=True)
                    dw = _wgrad(w, dyq_t, xq_t, T)
        else:
            xt_data, xt_inv, wt_data, wt_inv, w = ctx.saved_tensors
            xq_t = f8.Fp8Tensor(xt_data, T, xt_inv, False)
            wq_t = f8.Fp8Tensor(wt_data, w.shape[0], wt_inv, False)
            need_t = ctx.needs_input_grad[1]
            dyq, dyq_t = f8.quantize_fp8(dy2, f8.PER_TENSOR, e5m2=True, want_t=need_t)
            if ctx.needs_input_grad[0]:
                dx = f8.matmul_fp8(dyq, wq_t, out_dtype=ctx.act_dtype).view(ctx.x_shape)
            if need_t:
                dw = _wgrad(w, dyq_t, xq_t, T)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None


class Float8Linear(nn.Linear):
    recipe = "rowwise"

    def forward(self, x):
        if x.numel() == 0:
            return torch.nn.functional.linear(x, self.weight, self.bias)
        return _Fp8Linear.apply(x, self.weight, self.bias, self.recipe != "tensorwise",
                                self.recipe == "rowwise_with_gw_hp")


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
