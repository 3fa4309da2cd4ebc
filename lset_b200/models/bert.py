"""BERT / XLM-RoBERTa post-LayerNorm encoder on the flat-stream kernels.

State-dict keys follow the reference (lset/models/encoder/bert/model.py:14-142):
``embeddings.{word,position,token_type}_embeddings.weight``, ``embeddings.LayerNorm.*``,
``layers.{i}.attention.{query,key,value,dense}.*`` (or ``qkv_proj`` when fused),
``layers.{i}.attention.LayerNorm.*``, ``layers.{i}.mlp.{dense_in,dense_out}.*``,
``layers.{i}.mlp.LayerNorm.*``. Attention is bidirectional; padding is skipped through the plan.
"""
from __future__ import annotations


import torch
import torch.nn as nn

from ..ops import activation as act_ops
from ..ops import attention as attn_ops
from ..ops import embedding as emb_ops
from ..ops import norm as norm_ops
from .configs import BertConfig
from .layers import Linear, StreamCtx, make_stream_ctx


class BertEmbeddings(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        H = config.hidden_size
        self.word_embeddings = nn.Embedding(config.vocab_size, H, padding_idx=config.pad_token_id)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings, H)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, H)
        self.LayerNorm = nn.LayerNorm(H, eps=config.layer_norm_eps)
        self.position_offset = config.position_offset

    def forward(self, flat_ids, flat_pos, flat_types=None):
        if flat_types is None:
            flat_types = torch.zeros_like(flat_ids)
        x = emb_ops.embedding(
            flat_ids, self.word_embeddings.weight,
            extra=((flat_pos + self.position_offset, self.position_embeddings.weight),
                   (flat_types, self.token_type_embeddings.weight)))
        ln = self.LayerNorm
        return norm_ops.layer_norm(x, ln.weight, ln.bias, ln.eps)


class BertAttention(nn.Module):
    def __init__(self, config: BertConfig, fused_qkv: bool = False):
        super().__init__()
        H = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = H // config.num_attention_heads
        self.fused_qkv = fused_qkv
        if fused_qkv:
            self.qkv_proj = Linear(H, 3 * H)
        else:
            self.query, self.key, self.value = Linear(H, H), Linear(H, H), Linear(H, H)
        self.dense = Linear(H, H)
        self.LayerNorm = nn.LayerNorm(H, eps=config.layer_norm_eps)

    def forward(self, x, ctx: StreamCtx):
        T, hd = x.shape[0], self.head_dim
        if self.fused_qkv:
            qkv = self.qkv_proj(x).view(T, -1, hd)
            nh = qkv.shape[1] // 3
            q, k, v = qkv[:, :nh], qkv[:, nh:2 * nh], qkv[:, 2 * nh:]
        else:
            q = self.query(x).view(T, -1, hd)
            k = self.key(x).view(T, -1, hd)
            v = self.value(x).view(T, -1, hd)
        o = attn_ops.varlen_attention(q, k, v, ctx.plan, causal=False)
        out = self.dense(o.reshape(T, -1))
        ln = self.LayerNorm
        y, _ = norm_ops.residual_layer_norm(x, out, ln.weight, ln.bias, ln.eps)
        return y


class BertMLP(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.dense_in = Linear(config.hidden_size, config.intermediate_size)
        self.dense_out = Linear(config.intermediate_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, x):
        h = self.dense_out(act_ops.gelu(self.dense_in(x)))
        ln = self.LayerNorm
        y, _ = norm_ops.residual_layer_norm(x, h, ln.weight, ln.bias, ln.eps)
        return y


class BertBlock(nn.Module):
    def __init__(self, config: BertConfig, fused_qkv: bool = False):
        super().__init__()
        self.attention = BertAttention(config, fused_qkv)
        self.mlp = BertMLP(config)

    def forward(self, x, ctx: StreamCtx):
        return self.mlp(self.attention(x, ctx))


class BertEncoder(nn.Module):
    def __init__(self, config: BertConfig, fused_projections: bool = False):
        super().__init__()
        self.config = config
        self.fused_projections = fused_projections
        self.embeddings = BertEmbeddings(config)
        self.layers = nn.ModuleList(
            [BertBlock(config, fused_projections) for _ in range(config.num_hidden_layers)])

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, *, position_ids=None,
                cu_seqlens=None, max_seqlen=None, **_unused):
        dev = self.embeddings.word_embeddings.weight.device
        input_ids, attention_mask, token_type_ids, position_ids, cu_seqlens = (
            t.to(dev) if torch.is_tensor(t) and t.device != dev else t
            for t in (input_ids, attention_mask, token_type_ids, position_ids, cu_seqlens))
        ctx = make_stream_ctx(input_ids, attention_mask, position_ids, cu_seqlens, max_seqlen)
        types = token_type_ids.reshape(-1) if token_type_ids is not None else None
        x = self.embeddings(input_ids.reshape(-1), ctx.pos, types)
        for layer in self.layers:
            x = layer(x, ctx)
        if ctx.padded_shape is not None:
            x = x.view(*ctx.padded_shape, x.shape[-1])
        return {"hidden_states": x}

    def forward_packed(self, input_ids, position_ids, cu_seqlens, max_seqlen):
        return self(input_ids, position_ids=position_ids, cu_seqlens=cu_seqlens,
                    max_seqlen=max_seqlen)
