"""NF4 (4-bit NormalFloat) weight quantisation for QLoRA, implemented here directly (the reference
delegates to torchao's ``to_nf4``, lset/train/quantization/nf4.py:8-31): block-wise absmax scaling
to the 16 NF4 levels, with the fp32 block scales themselves quantised to int8 in groups of
``scaler_block_size`` (double quantisation). ``NF4Linear`` stores the packed codes as buffers and
dequantises to bf16 for the GEMM; it has no trainable parameters.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops.gemm import linear as gemm_linear

NF4_LEVELS = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
    0.7229568362236023, 1.0])


def _pick_scaler_block(n_blocks: int, want: int) -> int:
    b = 1
    while b * 2 <= want and n_blocks % (b * 2) == 0:
        b *= 2
    return b


def to_nf4(weight: torch.Tensor, block_size: int = 64, scaler_block_size: int = 256) -> dict:
    """Quantise a 2-D weight. Returns the packed representation as a dict of tensors."""
    w = weight.detach().float().reshape(-1)
    if w.numel() % block_size != 0:
        raise ValueError(f"weight size {w.numel()} is not a multiple of block_size {block_size}")
    blocks = w.view(-1, block_size)
    absmax = blocks.abs().amax(dim=1).clamp(min=1e-12)
    levels = NF4_LEVELS.to(w.device)
    codes = ((blocks / absmax[:, None])[..., None] - levels).abs().argmin(dim=-1).to(torch.uint8)
    packed = (codes[:, 0::2] << 4) | codes[:, 1::2]
    sb = _pick_scaler_block(absmax.numel(), scaler_block_size)
    mean = absmax.mean()
    groups = (absmax - mean).view(-1, sb)
    gmax = groups.abs().amax(dim=1).clamp(min=1e-12)
    q_scales = torch.round(groups / gmax[:, None] * 127.0).to(torch.int8)
    return {"packed": packed.reshape(-1), "q_scales": q_scales.reshape(-1), "scale_absmax": gmax,
            "scale_mean": mean.reshape(1), "shape": torch.tensor(weight.shape),
            "block_size": torch.tensor(block_size), "scaler_block_size": torch.tensor(sb)}


def from_nf4(q: dict, dtype=torch.bfloat16) -> torch.Tensor:
    bs, sb = int(q["block_size"]), int(q["scaler_block_size"])
    absmax = (q["q_scales"].float().view(-1, sb) / 127.0 * q["scale_absmax"][:, None]).reshape(-1) \
        + q["scale_mean"]
    packed = q["packed"].view(-1, bs // 2)
    codes = torch.stack([(packed >> 4) & 0xF, packed & 0xF], dim=-1).reshape(-1, bs).long()
    vals = NF4_LEVELS.to(packed.device)[codes] * absmax[:, None]
    return vals.reshape(tuple(int(s) for s in q["shape"])).to(dtype)


class NF4Linear(nn.Linear):
    """Frozen linear layer whose weight lives as NF4 codes."""

    def __init__(self, in_features, out_features, q: dict, bias=None, compute_dtype=torch.bfloat16):
        nn.Module.__init__(self)
        self.in_features, self.out_features = in_features, out_features
        self.compute_dtype = compute_dtype
        for k, v in q.items():
            self.register_buffer(f"nf4_{k}", v)
        self.register_buffer("bias_buf", bias)

    def _q(self) -> dict:
        return {k[4:]: v for k, v in self._buffers.items() if k.startswith("nf4_")}

    def dequantized_weight(self) -> torch.Tensor:
        return from_nf4(self._q(), self.compute_dtype)

    @property
    def weight(self):
        return self.dequantized_weight()

    @property
    def bias(self):
        return self._buffers.get("bias_buf")

    def forward(self, x):
        return gemm_linear(x, self.dequantized_weight().to(x.dtype), self.bias)


def quantize_linear_nf4(module: nn.Linear, block_size: int = 64, scaler_block_size: int = 256) -> NF4Linear:
    q = to_nf4(module.weight.data, block_size, scaler_block_size)
    dt = module.weight.dtype if module.weight.dtype != torch.float32 else torch.float32
    bias = module.bias.data.clone() if module.bias is not None else None
    return NF4Linear(module.in_features, module.out_features, q, bias, compute_dtype=dt)
