"""Decoder-style embedders: Qwen3 (causal, QK-norm), bidirectional Llama, EmbeddingGemma.

One implementation, configured by ``DecoderTraits``; the three public classes only pick traits.
Blocks keep the residual stream open across block boundaries so that ``residual + branch_output``
is always fused with the following RMSNorm (the structure of lset/models/decoder/qwen3/block.py:39-68
and, for Gemma's four norms per block, lset/models/decoder/gemma/model.py:195-202).

``forward(input_ids, attention_mask=None, return_lm_logits=False, *, position_ids=None,
cu_seqlens=None, max_seqlen=None) -> {"hidden_states"[, "lm_logits"]}`` accepts padded ``[B, S]``
batches or a packed stream (``cu_seqlens`` given); ``forward_packed`` is the packed shorthand.
Unlike the reference's Gemma model (lset/models/decoder/gemma/model.py:245-273) every family has a
packed path here, because all of them run on the same flat-stream kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..ops import block as block_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from .configs import GemmaConfig, LlamaConfig, Qwen3Config
from .layers import Attention, Embedding, GatedMLP, RMSNorm, StreamCtx, make_stream_ctx


@dataclass
class DecoderTraits:
    causal: bool = True
    qk_norm: bool = False
    unit_offset_norm: bool = False      # Gemma "(1 + w)" norms
    activation: str = "swiglu"
    sandwich_norms: bool = False        # Gemma: post-attention and post-feedforward norms as well
    embed_scale: float = 1.0
    softmax_scale: Optional[float] = None


class DecoderBlock(nn.Module):
    def __init__(self, config, traits: DecoderTraits, layer_idx: int, fused_projections: bool):
        super().__init__()
        H, eps, uo = config.hidden_size, config.rms_norm_eps, traits.unit_offset_norm
        theta = config.rope_theta
        if traits.sandwich_norms:
            types = getattr(config, "layer_types", None) or []
            if layer_idx < len(types) and types[layer_idx] == "sliding_attention":
                theta = config.rope_local_base_freq
        self.traits = traits
        self.input_layernorm = RMSNorm(H, eps, uo)
        self.self_attn = Attention(
            H, config.num_attention_heads, config.num_key_value_heads, config.head_dim,
            causal=traits.causal, qk_norm=traits.qk_norm, norm_eps=eps, norm_unit_offset=uo,
            bias=getattr(config, "attention_bias", False), fused_qkv=fused_projections,
            rope_theta=theta, rope_scaling=getattr(config, "rope_scaling", None),
            softmax_scale=traits.softmax_scale)
        self.post_attention_layernorm = RMSNorm(H, eps, uo)
        if traits.sandwich_norms:
            self.pre_feedforward_layernorm = RMSNorm(H, eps, uo)
        self.mlp = GatedMLP(H, config.intermediate_size, traits.activation, fused_projections)
        if traits.sandwich_norms:
            self.post_feedforward_layernorm = RMSNorm(H, eps, uo)

    def forward(self, branch, residual, ctx: StreamCtx, prev_post_norm: Optional[RMSNorm] = None):
        """``branch`` is the previous block's un-added output (or the embeddings for block 0).
        Returns ``(branch_out, residual)`` with the final add left to the next norm."""
        if prev_post_norm is None and block_ops.usable(self, branch, ctx):
            return block_ops.run(self, branch, residual, ctx)   # the whole block in one native call
        n_in, n_post = self.input_layernorm, self.post_attention_layernorm
        if residual is None:
            x, residual = n_in(branch), branch
        elif prev_post_norm is not None:  # Gemma: post-feedforward norm, add, input norm
            x, residual = norm_ops.double_residual_rms_norm(
                residual, branch, prev_post_norm.weight, n_in.weight, n_in.eps, n_in.w_off)
        else:
            x, residual = norm_ops.residual_rms_norm(residual, branch, n_in.weight, n_in.eps, n_in.w_off)
        a = self.self_attn(x, ctx)
        if self.traits.sandwich_norms:
            n_pre = self.pre_feedforward_layernorm
            x, residual = norm_ops.double_residual_rms_norm(
                residual, a, n_post.weight, n_pre.weight, n_pre.eps, n_pre.w_off)
        else:
            x, residual = norm_ops.residual_rms_norm(residual, a, n_post.weight, n_post.eps, n_post.w_off)
        return self.mlp(x), residual


class DecoderModel(nn.Module):
    traits = DecoderTraits()

    def __init__(self, config, fused_projections: bool = False, traits: Optional[DecoderTraits] = None):
        super().__init__()
        self.config = config
        self.fused_projections = fused_projections
        if traits is not None:
            self.traits = traits
        t = self.traits
        self.embed_tokens = Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(
            [DecoderBlock(config, t, i, fused_projections) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, t.unit_offset_norm)

    # ------------------------------------------------------------------ API
    def forward(self, input_ids, attention_mask=None, return_lm_logits: bool = False, *,
                position_ids=None, cu_seqlens=None, max_seqlen=None, **_unused):
        dev = self.embed_tokens.weight.device
        input_ids, attention_mask, position_ids, cu_seqlens = (
            t.to(dev) if torch.is_tensor(t) and t.device != dev else t
            for t in (input_ids, attention_mask, position_ids, cu_seqlens))
        ctx = make_stream_ctx(input_ids, attention_mask, position_ids, cu_seqlens, max_seqlen)
        hidden = self._run(input_ids.reshape(-1), ctx)
        if ctx.padded_shape is not None:
            hidden = hidden.view(*ctx.padded_shape, hidden.shape[-1])
        out = {"hidden_states": hidden}
        if return_lm_logits:
            out["lm_logits"] = gemm_ops.linear(hidden, self.embed_tokens.weight)
        return out

    def forward_packed(self, input_ids, position_ids, cu_seqlens, max_seqlen,
                       return_lm_logits: bool = False):
        return self(input_ids, return_lm_logits=return_lm_logits, position_ids=position_ids,
                    cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)

    # ------------------------------------------------------------------ core
    def _embed(self, flat_ids):
        from ..ops.embedding import embedding

        return embedding(flat_ids, self.embed_tokens.weight, scale=self.traits.embed_scale)

    _sp = None  # sequence-parallel state, set by ``lset_b200.dist.tp.apply_tp``

    def _run(self, flat_ids, ctx: StreamCtx):
        branch, residual = self._embed(flat_ids), None
        sp = self._sp
        if sp is not None:
            from ..dist import tp_fused

            T = branch.shape[0]
            branch = tp_fused.shard_tokens(branch, sp)  # blocks see this rank's tokens only
        prev_post = None
        for layer in self.layers:
            branch, residual = layer(branch, residual, ctx, prev_post)
            prev_post = layer.post_feedforward_layernorm if self.traits.sandwich_norms else None
        n = self.norm
        if prev_post is not None:
            hidden, _ = norm_ops.double_residual_rms_norm(
                residual, branch, prev_post.weight, n.weight, n.eps, n.w_off)
        else:
            hidden, _ = norm_ops.residual_rms_norm(residual, branch, n.weight, n.eps, n.w_off)
        if sp is not None:
            hidden = tp_fused.unshard_tokens(hidden, T, sp)
        return hidden


    def run_stage(self, flat_ids, stream, ctx: StreamCtx, lo: int, hi: int):
        """One pipeline stage: layers ``lo..hi-1``. The first stage (``lo == 0``) starts from the
        embeddings of ``flat_ids``; later stages take ``stream = (branch, residual)`` from the
        stage before. The last stage (``hi == len(layers)``) returns the final hidden states, the
        others the open residual stream ``(branch, residual)`` for the next stage."""
        if self.traits.sandwich_norms:
            raise NotImplementedError("pipeline stages are not available for sandwich-norm blocks")
        if lo == 0:
            branch, residual = self._embed(flat_ids), None
        else:
            branch, residual = stream
        for layer in list(self.layers)[lo:hi]:
            branch, residual = layer(branch, residual, ctx, None)
        if hi < len(self.layers):
            return branch, residual
        n = self.norm
        hidden, _ = norm_ops.residual_rms_norm(residual, branch, n.weight, n.eps, n.w_off)
        return hidden


class Qwen3Decoder(DecoderModel):
    """Qwen3 embedder: causal attention, per-head QK RMSNorm, SwiGLU."""

    traits = DecoderTraits(causal=True, qk_norm=True)

    def __init__(self, config: Qwen3Config, fused_projections: bool = False):
        super().__init__(config, fused_projections)


class LlamaBidirectionalModel(DecoderModel):
    """Llama backbone with bidirectional attention (llama-nemotron-embed / nv-embed style)."""

    traits = DecoderTraits(causal=False, qk_norm=False)

    def __init__(self, config: LlamaConfig, fused_projections: bool = False):
        super().__init__(config, fused_projections)


class EmbeddingGemmaModel(DecoderModel):
    """Gemma-3 text backbone as used by EmbeddingGemma: ``(1+w)`` norms, four norms per block,
    tanh-GeGLU, embeddings scaled by sqrt(H), query scaled by ``query_pre_attn_scalar**-0.5``,
    global / local RoPE bases per layer type, causal attention (the sliding window itself is not
    applied, as in lset/models/decoder/gemma/model.py:55-56,112-133)."""

    def __init__(self, config: GemmaConfig, fused_projections: bool = False):
        traits = DecoderTraits(
            causal=True, qk_norm=True, unit_offset_norm=True, activation="geglu",
            sandwich_norms=True, embed_scale=math.sqrt(config.hidden_size),
            softmax_scale=float(config.query_pre_attn_scalar) ** -0.5)
        super().__init__(config, fused_projections, traits)
