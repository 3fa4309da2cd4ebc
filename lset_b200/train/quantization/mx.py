"""MXFP8 training (cf. lset/train/quantization/mx.py:11-25): microscaling float8 — blocks of 32
values along the contraction dimension share one power-of-two (E8M0) scale. Emulated numerics on
the bf16 GEMM, like the reference's ``mxfp8_emulated`` recipe; the ``mxfp8_cublas*`` recipe names
are accepted and map to the same path."""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops.gemm import linear as gemm_linear

MX_RECIPES = ("mxfp8_emulated", "mxfp8_cublas", "mxfp8_cublas_rceil")
BLOCK = 32


def fake_quant_mxfp8(x: torch.Tensor, rceil: bool = False) -> torch.Tensor:
    shape = x.shape
    pad = (-shape[-1]) % BLOCK
    xf = torch.nn.functional.pad(x.float(), (0, pad)).reshape(-1, BLOCK)
    amax = xf.abs().amax(dim=1, keepdim=True).clamp(min=2.0 ** -126)
    e = torch.log2(amax / 448.0)
    exp = torch.ceil(e) if rceil else torch.floor(e) + 1
    scale = torch.exp2(exp)
    q = (xf / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * scale
    q = q.reshape(*shape[:-1], shape[-1] + pad)[..., : shape[-1]]
    return q.to(x.dtype)


class MXLinear(nn.Linear):
    rceil = False

    def forward(self, x):
        xq = x + (fake_quant_mxfp8(x, self.rceil) - x).detach()
        wq = self.weight + (fake_quant_mxfp8(self.weight, self.rceil) - self.weight).detach()
        return gemm_linear(xq, wq, self.bias)


def apply_mxfp8_training(model: nn.Module, recipe: str = "mxfp8_emulated") -> nn.Module:
    if recipe not in MX_RECIPES:
        raise ValueError(f"Unknown MX recipe {recipe!r}; choose from {MX_RECIPES}")
    for mod in model.modules():
        if isinstance(mod, nn.Linear) and type(mod).__name__ == "Linear" and mod.in_features % BLOCK == 0:
            mod.__class__ = MXLinear
            mod.rceil = recipe.endswith("rceil")
    return model
