"""Building blocks shared by every model family.

All models run on one flat token stream ``[T, H]``: a packed batch is used as is, a padded batch
``[B, S]`` is flattened and described by an attention plan that skips the padding. ``StreamCtx``
carries what every layer needs for one forward (plan, position ids, RoPE tables).

Module and parameter names match the reference's state-dict keys (``self_attn.q_proj.weight``,
``self_attn.q_norm.weight``, ``mlp.gate_proj.weight``, ``qkv_proj`` / ``gate_up_proj`` when fused;
lset/models/decoder/qwen3/attention.py:66-78, lset/models/decoder/qwen3/mlp.py:15-28).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn

from ..ops import activation as act_ops
from ..ops import attention as attn_ops
from ..ops import embedding as emb_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from ..ops import rope as rope_ops
from ..ops.runtime_options import enabled


class Linear(nn.Linear):
    """``nn.Linear`` whose forward runs the tcgen05 GEMM for bf16 CUDA tensors."""

    def forward(self, x):
        return gemm_ops.linear(x, self.weight, self.bias)


class Embedding(nn.Embedding):
    """``nn.Embedding`` whose forward runs the native gather kernel for bf16 CUDA tables."""

    def forward(self, ids):
        return emb_ops.embedding(ids, self.weight)


class RMSNorm(nn.Module):
    """RMSNorm; ``unit_offset`` selects Gemma's ``(1 + w)`` weight (initialised to zero)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, unit_offset: bool = False):
        super().__init__()
        self.eps = eps
        self.w_off = 1.0 if unit_offset else 0.0
        init = torch.zeros if unit_offset else torch.ones
        self.weight = nn.Parameter(init(hidden_size))

    def forward(self, x):
        return norm_ops.rms_norm(x, self.weight, self.eps, self.w_off)


@dataclass
class StreamCtx:
    """Per-forward context for a flat token stream."""

    plan: attn_ops.AttnPlan
    pos: torch.Tensor                      # [T] position ids
    max_pos: int
    padded_shape: Optional[tuple] = None   # (B, S) when the stream is a flattened padded batch
    tables: dict = field(default_factory=dict)

    def rope(self, head_dim: int, theta: float, scaling=None):
        key = (head_dim, theta, None if not scaling else tuple(sorted(scaling.items())))
        hit = self.tables.get(key)
        if hit is None:
            hit = rope_ops.rope_tables(head_dim, self.max_pos, theta, self.pos.device, scaling)
            self.tables[key] = hit
        return hit


def make_stream_ctx(input_ids, attention_mask=None, position_ids=None, cu_seqlens=None,
                    max_seqlen=None) -> StreamCtx:
    """Build the context for a packed (``cu_seqlens`` given) or padded ``[B, S]`` batch."""
    dev = input_ids.device
    if cu_seqlens is not None:
        T = input_ids.shape[0]
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
        plan = attn_ops.AttnPlan(cu_seqlens, max_seqlen, T)
        if position_ids is None:
            seg = torch.repeat_interleave(
                torch.arange(cu_seqlens.numel() - 1, device=dev),
                (cu_seqlens[1:] - cu_seqlens[:-1]).long(), output_size=T)
            position_ids = torch.arange(T, device=dev) - cu_seqlens[:-1].long()[seg]
        return StreamCtx(plan, position_ids, int(max_seqlen))
    B, S = input_ids.shape
    if attention_mask is None:
        cu = torch.arange(B + 1, device=dev, dtype=torch.int32) * S
        plan = attn_ops.AttnPlan(cu, S, B * S)
    else:
        plan = attn_ops.AttnPlan.from_mask(attention_mask)
    if position_ids is None:
        position_ids = torch.arange(S, device=dev).repeat(B)
    else:
        position_ids = position_ids.expand(B, S).reshape(-1)
    return StreamCtx(plan, position_ids, S, padded_shape=(B, S))


class Attention(nn.Module):
    """Multi-head / grouped-query attention with RoPE and optional per-head QK RMSNorm."""

    def __init__(self, hidden_size, num_heads, num_kv_heads, head_dim, *, causal, qk_norm,
                 norm_eps=1e-6, norm_unit_offset=False, bias=False, fused_qkv=False,
                 rope_theta=1e6, rope_scaling=None, softmax_scale=None):
        super().__init__()
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.causal = causal
        self.rope_theta, self.rope_scaling = rope_theta, rope_scaling
        self.softmax_scale = softmax_scale
        self.fused_qkv = fused_qkv
        q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        if fused_qkv:
            self.qkv_proj = Linear(hidden_size, q_dim + 2 * kv_dim, bias=bias)
        else:
            self.q_proj = Linear(hidden_size, q_dim, bias=bias)
            self.k_proj = Linear(hidden_size, kv_dim, bias=bias)
            self.v_proj = Linear(hidden_size, kv_dim, bias=bias)
        self.o_proj = Linear(q_dim, hidden_size, bias=bias)
        if qk_norm:
            self.q_norm = RMSNorm(head_dim, norm_eps, norm_unit_offset)
            self.k_norm = RMSNorm(head_dim, norm_eps, norm_unit_offset)
        else:
            self.q_norm = self.k_norm = None

    def forward(self, x, ctx: StreamCtx):
        # T is the full stream length: under sequence parallelism ``x`` holds only this rank's
        # tokens, the projections return every token (padded to a multiple of the group size) and
        # ``o_proj`` hands back a token shard again.
        T, hd = int(ctx.pos.shape[0]), self.head_dim
        cos, sin = ctx.rope(hd, self.rope_theta, self.rope_scaling)
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        eps = self.q_norm.eps if self.q_norm is not None else 1e-6
        w_off = self.q_norm.w_off if self.q_norm is not None else 0.0
        if self.fused_qkv:
            qkv = self.qkv_proj(x)
            Tp = qkv.shape[0]
            # head counts come from the local weight shape so a tensor-parallel shard just works
            per = self.num_heads // self.num_kv_heads
            Hk = qkv.shape[-1] // ((per + 2) * hd)
            Hq = Hk * per
            if Tp != T:   # padded token shards (sequence parallelism); a full-range slice would
                qkv = qkv[:T]  # still cost a zero-fill and a copy in the backward
            o = attn_ops.qkv_attention(qkv.view(T, Hq + 2 * Hk, hd), qw, kw, cos, sin, ctx.pos,
                                       ctx.plan, Hq, Hk, self.causal, self.softmax_scale, eps, w_off)
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
            Tp = q.shape[0]
            if Tp != T:
                q, k, v = q[:T], k[:T], v[:T]
            q, k, v = q.view(T, -1, hd), k.view(T, -1, hd), v.view(T, -1, hd)
            Hq = q.shape[1]
            q, k = rope_ops.qk_norm_rope(q, k, qw, kw, cos, sin, ctx.pos, eps, w_off)
            o = attn_ops.varlen_attention(q, k, v, ctx.plan, self.causal, self.softmax_scale)
        o = o.reshape(T, Hq * hd)
        if Tp != T:
            o = torch.cat([o, o.new_zeros(Tp - T, o.shape[1])], dim=0)
        return self.o_proj(o)


class GatedMLP(nn.Module):
    """``down(act(gate(x)) * up(x))`` with SwiGLU (``swiglu``) or tanh-GeGLU (``geglu``)."""

    def __init__(self, hidden_size, intermediate_size, kind="swiglu", fused_gate_up=False):
        super().__init__()
        self.kind = kind
        self.fused_gate_up = fused_gate_up
        if fused_gate_up:
            self.gate_up_proj = Linear(hidden_size, 2 * intermediate_size, bias=False)
        else:
            self.gate_proj = Linear(hidden_size, intermediate_size, bias=False)
            self.up_proj = Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        if self.fused_gate_up:
            gu = self.gate_up_proj
            # plain bf16 projection on the GPU: the activation rides in the GEMM epilogue; wrapped
            # layers (tensor parallel, LoRA, quantised) go through their own forward
            if (type(gu) is Linear and gu.bias is None and "forward" not in gu.__dict__
                    and gemm_ops.linear_glu_supported(x, gu.weight) and enabled("fused_glu_gemm")):
                h = gemm_ops.linear_glu(x, gu.weight, self.kind)
                return self.down_proj(h)
            h = act_ops.glu(gu(x), self.kind)
        elif self.kind == "swiglu":
            h = act_ops.swiglu(self.gate_proj(x), self.up_proj(x))
        else:
            h = act_ops.geglu(self.gate_proj(x), self.up_proj(x))
        return self.down_proj(h)


def init_normal_(module: nn.Module, std: float = 0.02) -> None:
    """N(0, std) for matrices and embeddings; norm weights and biases keep their defaults."""
    for m in module.modules():
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=std)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)
