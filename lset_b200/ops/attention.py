"""Varlen (packed) attention on the native tcgen05 kernels, plus the eager oracle.

``AttnPlan`` is built once per packed batch from ``cu_seqlens`` (a device-side planning kernel, no
host sync) and reused by every layer's forward and backward. Padded batches are handled by the
same kernels: a ``[B, S]`` batch is a packed stream with ``cu_seqlens = arange(B+1) * S`` when
there is no padding, or is packed by its attention mask.

Replaces flash_attn_varlen_func / torch varlen_attn / SDPA of the reference
(lset/models/decoder/qwen3/attention.py:112-115,169-272).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _native as nv
from ._ac import run_expensive
from .runtime_options import options as _rt


class AttnPlan:
    """Tile lists for one packed batch. ``cu_seqlens``: int32 ``[B+1]`` on the device."""

    def __init__(self, cu_seqlens: torch.Tensor, max_seqlen: int, total_tokens: int,
                 seq_start: torch.Tensor | None = None, seq_end: torch.Tensor | None = None):
        self.cu_seqlens = cu_seqlens.to(torch.int32).contiguous() if cu_seqlens is not None else None
        if seq_start is None:
            # packed stream: sequence b is [cu[b], cu[b+1])
            seq_start, seq_end = self.cu_seqlens[:-1], self.cu_seqlens[1:]
        self.seq_start = seq_start.to(torch.int32)
        self.seq_end = seq_end.to(torch.int32)
        assert self.seq_start.stride(0) == 1 and self.seq_end.stride(0) == 1
        self.max_seqlen = int(max_seqlen)
        self.T = int(total_tokens)
        self.B = int(self.seq_start.numel())
        self._plans = {}

    @classmethod
    def from_mask(cls, attention_mask: torch.Tensor) -> "AttnPlan":
        """Plan for a padded ``[B, S]`` batch flattened to ``B*S`` tokens: every row is one sequence
        that covers only its unmasked (contiguous) span, left- or right-padded. No host sync."""
        B, S = attention_mask.shape
        m = attention_mask.to(torch.int32)
        lens = m.sum(1, dtype=torch.int32)
        first = torch.argmax(m, dim=1).to(torch.int32)
        base = torch.arange(B, device=m.device, dtype=torch.int32) * S
        start = (base + first).contiguous()
        return cls(None, S, B * S, seq_start=start, seq_end=(start + lens).contiguous())

    def tiles(self, tile_tokens: int):
        """(plan tensor, capacity) for a tile of ``tile_tokens`` tokens."""
        hit = self._plans.get(tile_tokens)
        if hit is not None:
            return hit
        cap = (self.T + tile_tokens - 1) // tile_tokens + self.B
        # two spare words behind the entries: the work counter of the persistent forward kernel and
        # the end of the last sequence (rows behind it are cleared by the attention launchers)
        plan = torch.empty(1 + 2 * cap + 2, dtype=torch.int32, device=self.seq_start.device)
        rc = nv.load().lb_attn_plan(nv.c_void_p(self.seq_start.data_ptr()),
                                    nv.c_void_p(self.seq_end.data_ptr()), nv.c_int(self.B),
                                    nv.c_int(tile_tokens), nv.c_void_p(plan.data_ptr()),
                                    nv.c_int(cap), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_attn_plan")
        nv.count_launch()
        self._plans[tile_tokens] = (plan, cap)
        return plan, cap


def attention_ref(q, k, v, cu_seqlens, causal: bool, scale: float | None = None, seq_end=None):
    """Eager oracle: per-sequence softmax attention in fp32. q: [T,Hq,hd]; k, v: [T,Hk,hd].
    Sequences are ``[cu[b], cu[b+1])``, or ``[cu_seqlens[b], seq_end[b])`` when ``seq_end`` is given;
    tokens outside every sequence get zeros."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    out = torch.zeros(T, Hq, hd, dtype=q.dtype, device=q.device)
    if seq_end is None:
        cu = cu_seqlens.tolist()
        spans = list(zip(cu[:-1], cu[1:]))
    else:
        spans = list(zip(cu_seqlens.tolist(), seq_end.tolist()))
    rep = Hq // Hk
    for s, e in spans:
        if e <= s:
            continue
        qs = q[s:e].float().transpose(0, 1)
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        att = torch.matmul(qs, ks.transpose(1, 2)) * scale
        if causal:
            L = e - s
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            att = att.masked_fill(~mask, float("-inf"))
        out[s:e] = torch.matmul(att.softmax(-1), vs).transpose(0, 1).to(q.dtype)
    return out


def _native_fwd(q, k, v, plan: AttnPlan, causal, scale):
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    G = Hq // Hk
    ptiles, cap = plan.tiles(128 // G)
    # tokens outside every sequence (padding) are never written by the kernel: keep them zero
    o = (torch.empty if plan.cu_seqlens is not None else torch.zeros)(
        T, Hq, hd, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
    rc = nv.load().lb_attn_fwd(
        nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), nv.c_void_p(k.data_ptr()),
        nv.c_ll(k.stride(0)), nv.c_void_p(v.data_ptr()), nv.c_ll(v.stride(0)),
        nv.c_void_p(plan.seq_start.data_ptr()), nv.c_void_p(plan.seq_end.data_ptr()),
        nv.c_void_p(ptiles.data_ptr()), nv.c_int(cap),
        nv.c_void_p(o.data_ptr()), nv.c_ll(Hq * hd), nv.c_void_p(lse.data_ptr()), nv.c_int(T),
        nv.c_int(Hq), nv.c_int(Hk), nv.c_int(hd), nv.c_float(scale), nv.c_int(int(causal)),
        nv.c_void_p(nv.status_word(q.device).data_ptr()), nv.c_void_p(nv.stream_ptr()))
    nv.check_rc(rc, "lb_attn_fwd")
    nv.count_launch(2)
    return o, lse


def _native_bwd(do, q, k, v, o, lse, plan: AttnPlan, causal, scale, dq, dk, dv):
    """Writes dq [T,Hq,hd], dk, dv [T,Hk,hd] (strided views allowed, unit inner stride)."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    G = Hq // Hk
    lib = nv.load()
    delta = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
    ptq, capq = plan.tiles(128 // G)
    ptk, capk = plan.tiles(128)
    rc = lib.lb_attn_bwd(
        nv.c_void_p(do.data_ptr()), nv.c_ll(do.stride(0)), nv.c_void_p(q.data_ptr()),
        nv.c_ll(q.stride(0)), nv.c_void_p(k.data_ptr()), nv.c_ll(k.stride(0)),
        nv.c_void_p(v.data_ptr()), nv.c_ll(v.stride(0)), nv.c_void_p(o.data_ptr()),
        nv.c_ll(o.stride(0)), nv.c_void_p(lse.data_ptr()), nv.c_void_p(delta.data_ptr()),
        nv.c_void_p(plan.seq_start.data_ptr()), nv.c_void_p(plan.seq_end.data_ptr()),
        nv.c_void_p(ptq.data_ptr()), nv.c_int(capq),
        nv.c_void_p(ptk.data_ptr()), nv.c_int(capk), nv.c_void_p(dq.data_ptr()),
        nv.c_ll(dq.stride(0)), nv.c_void_p(dk.data_ptr()), nv.c_ll(dk.stride(0)),
        nv.c_void_p(dv.data_ptr()), nv.c_ll(dv.stride(0)), nv.c_int(T), nv.c_int(Hq), nv.c_int(Hk),
        nv.c_int(hd), nv.c_float(scale), nv.c_int(int(causal)),
        nv.c_void_p(nv.status_word(q.device).data_ptr()), nv.c_void_p(nv.stream_ptr()))
    nv.check_rc(rc, "lb_attn_bwd")
    nv.count_launch(4)


def _unit_inner(t):
    return t if (t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0) \
        else t.contiguous()


class _VarlenAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, plan, causal, scale):
        q, k, v = _unit_inner(q), _unit_inner(k), _unit_inner(v)
        o, lse = run_expensive(lambda: _native_fwd(q, k, v, plan, causal, scale))
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.plan, ctx.causal, ctx.scale = plan, causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        do = do if do.is_contiguous() else do.contiguous()
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        _native_bwd(do, q, k, v, o, lse, ctx.plan, ctx.causal, ctx.scale, dq, dk, dv)
        return dq, dk, dv, None, None, None


class _QkvAttention(torch.autograd.Function):
    """Fused path for a fused QKV projection output ``qkv [T, Hq + 2Hk, hd]``: per-head RMSNorm +
    RoPE on q and k, then attention. The backward writes one ``dqkv`` buffer, so the projection's
    dgrad/wgrad GEMMs consume it without any slicing or concatenation."""

    @staticmethod
    def forward(ctx, qkv, qw, kw, cos, sin, pos, plan, Hq, Hk, causal, scale, eps, w_off):
        from .rope import rope_fwd_native

        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hk], qkv[:, Hq + Hk:]
        q_r, k_r, q_rstd, k_rstd = rope_fwd_native(q, k, qw, kw, cos, sin, pos, eps, w_off)
        o, lse = run_expensive(lambda: _native_fwd(q_r, k_r, v, plan, causal, scale))
        ctx.save_for_backward(qkv, qw, kw, cos, sin, pos, q_r, k_r, q_rstd, k_rstd, o, lse)
        ctx.meta = (plan, Hq, Hk, causal, scale, w_off)
        return o

    @staticmethod
    def backward(ctx, do):
        from .rope import deliver_norm_wgrads, rope_bwd_native

        qkv, qw, kw, cos, sin, pos, q_r, k_r, q_rstd, k_rstd, o, lse = ctx.saved_tensors
        plan, Hq, Hk, causal, scale, w_off = ctx.meta
        T, _, hd = qkv.shape
        do = do if do.is_contiguous() else do.contiguous()
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hk], qkv[:, Hq + Hk:]
        dqkv = torch.empty_like(qkv) if plan.cu_seqlens is not None else torch.zeros_like(qkv)
        dq_r = torch.empty(T, Hq, hd, dtype=qkv.dtype, device=qkv.device)
        dk_r = torch.empty(T, Hk, hd, dtype=qkv.dtype, device=qkv.device)
        if plan.cu_seqlens is None:
            dq_r.zero_()
            dk_r.zero_()
        _native_bwd(do, q_r, k_r, v, o, lse, plan, causal, scale, dq_r, dk_r, dqkv[:, Hq + Hk:])
        dwb = rope_bwd_native(dq_r, dk_r, q, k, qw, kw, cos, sin, pos, q_rstd, k_rstd, w_off,
                              dqkv[:, :Hq], dqkv[:, Hq:Hq + Hk])
        dqw, dkw = deliver_norm_wgrads(qw, kw, dwb, hd)
        return dqkv, dqw, dkw, None, None, None, None, None, None, None, None, None, None


def qkv_attention(qkv, qw, kw, cos, sin, pos, plan: AttnPlan, Hq: int, Hk: int, causal: bool,
                  scale: float | None = None, eps: float = 1e-6, w_off: float = 0.0):
    """RoPE (with per-head RMSNorm when ``qw`` is given) + attention on a fused ``[T, Hq+2Hk, hd]``
    projection output. Returns ``[T, Hq, hd]``."""
    from .rope import qk_norm_rope

    hd = qkv.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hk], qkv[:, Hq + Hk:]
    needs_grad = torch.is_grad_enabled() and qkv.requires_grad
    if native_supported(q, k) and qkv.is_contiguous() and not (needs_grad and hd > 128):
        return _QkvAttention.apply(qkv, qw, kw, cos, sin, pos, plan, Hq, Hk, bool(causal),
                                   float(scale), float(eps), float(w_off))
    q, k = qk_norm_rope(q, k, qw, kw, cos, sin, pos, eps, w_off)
    return varlen_attention(q, k, v, plan, causal, scale)


def native_supported(q, k) -> bool:
    if _rt.attention_backend == "sdpa":
        return False
    if not (nv.use_native(q, k) and q.dtype == torch.bfloat16):
        return False
    Hq, hd = q.shape[1], q.shape[2]
    Hk = k.shape[1]
    return hd in (64, 128, 256) and Hq % Hk == 0 and (Hq // Hk) in (1, 2, 4, 8)


def varlen_attention(q, k, v, plan: AttnPlan, causal: bool, scale: float | None = None):
    """Attention over a packed token stream. q: ``[T,Hq,hd]``, k/v: ``[T,Hk,hd]``; sequences are
    delimited by ``plan.cu_seqlens``. Returns ``[T,Hq,hd]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    # The dK/dV kernel keeps two head_dim-wide accumulators in TMEM: head_dim 256 does not fit, so
    # training at that width runs the eager path (inference still uses the native forward).
    if native_supported(q, k) and not (needs_grad and q.shape[-1] > 128):
        return _VarlenAttn.apply(q, k, v, plan, bool(causal), float(scale))
    if plan.cu_seqlens is None and not q.is_cuda and plan.B > 0 and plan.T % plan.B == 0:
        # CPU, padded [B, S] batch: one batched masked attention instead of a Python loop over the
        # sequences (rows of padding tokens are zeroed like in the per-sequence form)
        B, S = plan.B, plan.T // plan.B
        pos = torch.arange(S, device=q.device)[None, :] + torch.arange(B, device=q.device)[:, None] * S
        mask = (pos >= plan.seq_start[:, None]) & (pos < plan.seq_end[:, None])
        out = padded_attention_ref(q.view(B, S, *q.shape[1:]), k.view(B, S, *k.shape[1:]),
                                   v.view(B, S, *v.shape[1:]), mask, causal, scale)
        return (out * mask[:, :, None, None].to(out.dtype)).reshape(plan.T, *q.shape[1:])
    return attention_ref(q, k, v, plan.seq_start, causal, scale, seq_end=plan.seq_end)


def padded_attention_ref(q, k, v, attn_mask, causal: bool, scale: float | None = None):
    """Oracle for padded batches. q: [B,S,Hq,hd]; k, v: [B,S,Hk,hd]; attn_mask: [B,S] 1 = token."""
    B, S, Hq, hd = q.shape
    Hk = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    qf = q.transpose(1, 2).float()
    kf = k.transpose(1, 2).float().repeat_interleave(Hq // Hk, dim=1)
    vf = v.transpose(1, 2).float().repeat_interleave(Hq // Hk, dim=1)
    att = torch.matmul(qf, kf.transpose(2, 3)) * scale
    neg = torch.finfo(torch.float32).min
    if causal:
        tri = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        att = att.masked_fill(~tri, neg)
    if attn_mask is not None:
        att = att.masked_fill(~attn_mask.bool()[:, None, None, :], neg)
    out = torch.matmul(att.softmax(-1), vf)
    return out.transpose(1, 2).to(q.dtype)
