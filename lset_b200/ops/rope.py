"""Rotary position embedding, alone or fused with per-head RMSNorm of Q and K.

Tables are fp32 ``[positions, head_dim/2]`` built once per (theta, head_dim, scaling) and cached;
the kernel gathers rows by position id. Counterpart of lset/kernels/qk_norm_rope.py and
lset/kernels/rope.py; the frequency scaling follows lset/models/decoder/llama/attention.py:33-55.
"""
from __future__ import annotations

import math

import torch

from . import _native as nv
from ._grads import main_grad_of
from .norm import scratch
from .runtime_options import enabled

_tables = {}


def rope_tables(head_dim: int, max_pos: int, theta: float, device, scaling: dict | None = None):
    """Return ``(cos, sin)`` fp32 tensors of shape ``[max_pos, head_dim // 2]`` (cached, grown)."""
    skey = tuple(sorted(scaling.items())) if scaling else None
    key = (head_dim, float(theta), str(device), skey)
    cur = _tables.get(key)
    if cur is not None and cur[0].shape[0] >= max_pos:
        return cur
    n = max(max_pos, 512)
    n = 1 << (n - 1).bit_length()
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = float(scaling.get("factor", 8.0))
        lo = float(scaling.get("low_freq_factor", 1.0))
        hi = float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
    ang = torch.outer(torch.arange(n, dtype=torch.float32), inv)
    cur = (ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous())
    _tables[key] = cur
    return cur


def _rotate_ref(x, cos, sin):
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def qk_norm_rope_ref(q, k, qw, kw, cos, sin, pos, eps=1e-6, w_off=0.0):
    """q: [T, Hq, hd], k: [T, Hk, hd]; cos/sin tables; pos: [T] position ids."""
    c = cos[pos.long()].unsqueeze(1)
    s = sin[pos.long()].unsqueeze(1)

    def norm(x, w):
        if w is None:
            return x.float()
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return (xf * rstd).to(x.dtype).float() * (w.float() + w_off)

    return (_rotate_ref(norm(q, qw), c, s).to(q.dtype), _rotate_ref(norm(k, kw), c, s).to(k.dtype))


def rope_fwd_native(q, k, qw, kw, cos, sin, pos, eps, w_off):
    """Raw launcher. q: [T,Hq,hd], k: [T,Hk,hd] (strided views allowed). Returns
    ``(q_out, k_out, q_rstd, k_rstd)`` with contiguous outputs."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    assert q.stride(2) == 1 and k.stride(2) == 1 and q.stride(1) == hd and k.stride(1) == hd
    do_norm = qw is not None
    q_out = torch.empty(T, Hq, hd, dtype=q.dtype, device=q.device)
    k_out = torch.empty(T, Hk, hd, dtype=k.dtype, device=k.device)
    q_rstd = torch.empty(T, Hq, dtype=torch.float32, device=q.device) if do_norm else None
    k_rstd = torch.empty(T, Hk, dtype=torch.float32, device=q.device) if do_norm else None
    rc = nv.load().lb_qk_norm_rope_fwd(
        nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), nv.c_void_p(k.data_ptr()),
        nv.c_ll(k.stride(0)), nv.c_void_p(nv.ptr(qw)), nv.c_void_p(nv.ptr(kw)),
        nv.c_void_p(cos.data_ptr()), nv.c_void_p(sin.data_ptr()), nv.c_void_p(pos.data_ptr()),
        nv.c_int(int(pos.dtype == torch.int64)), nv.c_int(1),
        nv.c_void_p(q_out.data_ptr()), nv.c_ll(Hq * hd), nv.c_void_p(k_out.data_ptr()),
        nv.c_ll(Hk * hd), nv.c_void_p(nv.ptr(q_rstd)), nv.c_void_p(nv.ptr(k_rstd)),
        nv.c_int(T), nv.c_int(Hq), nv.c_int(Hk), nv.c_int(hd), nv.c_float(eps),
        nv.c_float(w_off), nv.c_int(int(do_norm)), nv.c_void_p(nv.stream_ptr()))
    nv.check_rc(rc, "lb_qk_norm_rope_fwd")
    nv.count_launch()
    return q_out, k_out, q_rstd, k_rstd


def rope_bwd_native(dq, dk, q, k, qw, kw, cos, sin, pos, q_rstd, k_rstd, w_off, dq_in, dk_in):
    """Raw launcher. dq/dk: contiguous grads of the rotated outputs; dq_in/dk_in: destination views
    (unit inner stride). Returns the fp32 ``[2*hd]`` weight gradient (q then k) or None."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    do_norm = qw is not None
    lib = nv.load()
    rows = lib.lb_rope_bwd_partial_rows()
    scr = scratch("rope_bwd", rows * 2 * hd, q.device) if do_norm else None
    dwb = torch.empty(2 * hd, dtype=torch.float32, device=q.device) if do_norm else None
    rc = lib.lb_qk_norm_rope_bwd(
        nv.c_void_p(dq.data_ptr()), nv.c_ll(dq.stride(0)), nv.c_void_p(dk.data_ptr()),
        nv.c_ll(dk.stride(0)), nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)),
        nv.c_void_p(k.data_ptr()), nv.c_ll(k.stride(0)), nv.c_void_p(nv.ptr(qw)),
        nv.c_void_p(nv.ptr(kw)), nv.c_void_p(cos.data_ptr()), nv.c_void_p(sin.data_ptr()),
        nv.c_void_p(pos.data_ptr()), nv.c_int(int(pos.dtype == torch.int64)), nv.c_int(1),
        nv.c_void_p(nv.ptr(q_rstd)), nv.c_void_p(nv.ptr(k_rstd)),
        nv.c_void_p(dq_in.data_ptr()), nv.c_ll(dq_in.stride(0)), nv.c_void_p(dk_in.data_ptr()),
        nv.c_ll(dk_in.stride(0)), nv.c_void_p(nv.ptr(scr)), nv.c_void_p(nv.ptr(dwb)),
        nv.c_int(1), nv.c_int(0), nv.c_int(T), nv.c_int(Hq), nv.c_int(Hk), nv.c_int(hd),
        nv.c_float(w_off), nv.c_int(int(do_norm)), nv.c_void_p(nv.stream_ptr()))
    nv.check_rc(rc, "lb_qk_norm_rope_bwd")
    nv.count_launch(2 if do_norm else 1)
    return dwb


def deliver_norm_wgrads(qw, kw, dwb, hd):
    """Route the fp32 q/k norm-weight gradients to ``main_grad`` or return them as tensors."""
    dqw = dkw = None
    if dwb is None:
        return dqw, dkw
    for w, sl, is_q in ((qw, dwb[:hd], True), (kw, dwb[hd:], False)):
        mg = main_grad_of(w)
        if mg is not None:
            mg.add_(sl)
        elif is_q:
            dqw = sl.to(w.dtype)
        else:
            dkw = sl.to(w.dtype)
    return dqw, dkw


class _QkNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, qw, kw, cos, sin, pos, eps, w_off):
        q_out, k_out, q_rstd, k_rstd = rope_fwd_native(q, k, qw, kw, cos, sin, pos, eps, w_off)
        ctx.save_for_backward(q, k, qw, kw, cos, sin, pos, q_rstd, k_rstd)
        ctx.w_off = w_off
        return q_out, k_out

    @staticmethod
    def backward(ctx, dq, dk):
        q, k, qw, kw, cos, sin, pos, q_rstd, k_rstd = ctx.saved_tensors
        T, Hq, hd = q.shape
        Hk = k.shape[1]
        dq = dq if dq.is_contiguous() else dq.contiguous()
        dk = dk if dk.is_contiguous() else dk.contiguous()
        dqk = torch.empty(T, Hq + Hk, hd, dtype=q.dtype, device=q.device)
        dq_in, dk_in = dqk[:, :Hq], dqk[:, Hq:]
        dwb = rope_bwd_native(dq, dk, q, k, qw, kw, cos, sin, pos, q_rstd, k_rstd, ctx.w_off,
                              dq_in, dk_in)
        dqw, dkw = deliver_norm_wgrads(qw, kw, dwb, hd)
        return dq_in, dk_in, dqw, dkw, None, None, None, None, None


def qk_norm_rope(q, k, qw, kw, cos, sin, pos, eps=1e-6, w_off=0.0):
    """Per-head RMSNorm (skipped when ``qw`` is None) followed by RoPE on ``q [T,Hq,hd]`` and
    ``k [T,Hk,hd]``; ``pos [T]`` holds each token's position. Returns new ``(q, k)`` tensors."""
    native = (nv.use_native(q, k) and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128, 256)
              and enabled("fused_qk_norm_rope"))
    if not native:
        return qk_norm_rope_ref(q, k, qw, kw, cos, sin, pos, eps, w_off)
    return _QkNormRope.apply(q, k, qw, kw, cos, sin, pos, eps, w_off)


def apply_rope(q, k, cos, sin, pos):
    """RoPE only (Llama / Gemma without QK-norm fusion)."""
    return qk_norm_rope(q, k, None, None, cos, sin, pos)
