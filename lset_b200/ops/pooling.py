"""L2 normalisation and pooling over padded or packed hidden states.

``pool`` / ``packed_pool`` keep the reference's interface (lset/models/pooling.py:8-30,
lset/models/packed_pooling.py:10-48): strategies ``last_token`` (left padding), ``cls``, ``mean``,
``weighted_mean``. On CUDA bf16 tensors the packed paths run the gather+normalise and
segment-mean kernels; everything has an eager twin that serves as oracle and CPU path.
Normalisation is ``x / max(‖x‖, 1e-12)`` everywhere.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native as nv
from .runtime_options import enabled

_EPS = 1e-12


def _bf16_cuda(*ts):
    return enabled("fused_pool_normalize") and nv.use_native(*ts) and all(t.dtype == torch.bfloat16 for t in ts if t.is_floating_point())


class _GatherL2Norm(torch.autograd.Function):
    """out[m] = normalize(x[idx[m], :D]); idx None = identity. x: [N, ld] with unit inner stride."""

    @staticmethod
    def forward(ctx, x, idx, D, do_norm):
        M = x.shape[0] if idx is None else idx.shape[0]
        y = torch.empty(M, D, dtype=x.dtype, device=x.device)
        norm = torch.empty(M, dtype=torch.float32, device=x.device)
        rc = nv.load().lb_l2norm_fwd(
            nv.c_void_p(x.data_ptr()), nv.c_ll(x.stride(0)), nv.c_void_p(nv.ptr(idx)),
            nv.c_void_p(y.data_ptr()), nv.c_ll(D), nv.c_void_p(norm.data_ptr()), nv.c_int(M),
            nv.c_int(D), nv.c_float(_EPS), nv.c_int(int(do_norm)), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_l2norm_fwd")
        nv.count_launch()
        ctx.save_for_backward(y, norm, idx)
        ctx.x_shape = x.shape
        ctx.x_stride0 = x.stride(0)
        ctx.D = D
        ctx.do_norm = do_norm
        return y

    @staticmethod
    def backward(ctx, gy):
        y, norm, idx = ctx.saved_tensors
        M, D = y.shape
        gy = gy if gy.is_contiguous() else gy.contiguous()
        full = idx is not None or D != ctx.x_shape[1]
        dx = (torch.zeros if full else torch.empty)(ctx.x_shape, dtype=y.dtype, device=y.device)
        rc = nv.load().lb_l2norm_bwd(
            nv.c_void_p(gy.data_ptr()), nv.c_ll(D), nv.c_void_p(y.data_ptr()), nv.c_ll(D),
            nv.c_void_p(norm.data_ptr()), nv.c_void_p(nv.ptr(idx)), nv.c_void_p(dx.data_ptr()),
            nv.c_ll(dx.stride(0)), nv.c_int(M), nv.c_int(D), nv.c_int(int(ctx.do_norm)),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_l2norm_bwd")
        nv.count_launch()
        return dx, None, None, None


def normalize(x, dim: int = -1):
    """L2-normalise the last dimension."""
    if dim in (-1, x.dim() - 1) and _bf16_cuda(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.stride(1) == 1 and x2.stride(0) % 8 == 0 else x2.contiguous()
        return _GatherL2Norm.apply(x2, None, x2.shape[1], True).view(x.shape)
    return F.normalize(x.float(), p=2, dim=dim, eps=_EPS).to(x.dtype)


def gather_normalize(hidden, idx, do_norm=True):
    """Rows ``idx`` of ``hidden [T, H]`` (optionally L2-normalised) in one kernel."""
    if _bf16_cuda(hidden) and hidden.shape[-1] % 8 == 0 and hidden.shape[-1] <= 8192:
        h2 = hidden if hidden.stride(1) == 1 else hidden.contiguous()
        return _GatherL2Norm.apply(h2, idx.to(device=h2.device, dtype=torch.int64), h2.shape[1], do_norm)
    out = hidden[idx.long()]
    return normalize(out) if do_norm else out


class _SegmentMean(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu, weighted):
        M = cu.shape[0] - 1
        H = x.shape[1]
        out = torch.empty(M, H, dtype=x.dtype, device=x.device)
        rc = nv.load().lb_segment_mean_fwd(
            nv.c_void_p(x.data_ptr()), nv.c_void_p(cu.data_ptr()), nv.c_void_p(out.data_ptr()),
            nv.c_int(M), nv.c_int(H), nv.c_int(int(weighted)), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_segment_mean_fwd")
        nv.count_launch()
        ctx.save_for_backward(cu)
        ctx.T = x.shape[0]
        ctx.weighted = weighted
        return out

    @staticmethod
    def backward(ctx, g):
        (cu,) = ctx.saved_tensors
        M, H = g.shape
        g = g if g.is_contiguous() else g.contiguous()
        dx = torch.zeros(ctx.T, H, dtype=g.dtype, device=g.device)
        rc = nv.load().lb_segment_mean_bwd(
            nv.c_void_p(g.data_ptr()), nv.c_void_p(cu.data_ptr()), nv.c_void_p(dx.data_ptr()),
            nv.c_int(M), nv.c_int(H), nv.c_int(int(ctx.weighted)), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_segment_mean_bwd")
        nv.count_launch()
        return dx, None, None


def segment_mean_ref(hidden, cu_seqlens, weighted=False):
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
    M = lens.shape[0]
    seg = torch.repeat_interleave(torch.arange(M, device=hidden.device), lens)
    hf = hidden.float()
    if weighted:
        pos = torch.arange(hidden.shape[0], device=hidden.device) - cu_seqlens[:-1].long()[seg] + 1
        w = pos.float()
        den = torch.zeros(M, device=hidden.device).index_add_(0, seg, w)
        out = torch.zeros(M, hidden.shape[1], device=hidden.device).index_add_(0, seg, hf * w[:, None])
        return (out / den.clamp(min=1e-9)[:, None]).to(hidden.dtype)
    out = torch.zeros(M, hidden.shape[1], device=hidden.device).index_add_(0, seg, hf)
    return (out / lens.clamp(min=1).float()[:, None]).to(hidden.dtype)


def segment_mean(hidden, cu_seqlens, weighted=False):
    """Mean (or position-weighted mean) of each packed segment: ``[T, H] -> [M, H]``."""
    if _bf16_cuda(hidden) and hidden.shape[1] % 8 == 0 and hidden.shape[1] <= 8192:
        h2 = hidden if hidden.is_contiguous() else hidden.contiguous()
        return _SegmentMean.apply(h2, cu_seqlens.to(device=h2.device, dtype=torch.int32), weighted)
    return segment_mean_ref(hidden, cu_seqlens, weighted)


# --------------------------------------------------------------------------- public pooling API
def pool(hidden, attention_mask, strategy: str = "mean", normalize_output: bool = True):
    """Pool padded hidden states ``[B, S, H]`` with ``attention_mask [B, S]``."""
    if strategy == "last_token":
        out = hidden[:, -1]
    elif strategy == "cls":
        out = hidden[:, 0]
    elif strategy == "mean":
        m = attention_mask.unsqueeze(-1).to(torch.float32)
        out = ((hidden.float() * m).sum(1) / m.sum(1).clamp(min=1e-9)).to(hidden.dtype)
    elif strategy == "weighted_mean":
        m = attention_mask.to(torch.float32)
        w = torch.cumsum(m, dim=1) * m
        w = (w / w.sum(1, keepdim=True).clamp(min=1e-9)).unsqueeze(-1)
        out = (hidden.float() * w).sum(1).to(hidden.dtype)
    else:
        raise ValueError(f"Unknown pooling strategy: {strategy}")
    return normalize(out) if normalize_output else out


def packed_pool(hidden, cu_seqlens, strategy: str = "last_token", normalize_output: bool = True):
    """Pool packed hidden states ``[T, H]`` whose segments are given by ``cu_seqlens [M+1]``."""
    if strategy == "last_token":
        return gather_normalize(hidden, cu_seqlens[1:].long() - 1, normalize_output)
    if strategy == "cls":
        return gather_normalize(hidden, cu_seqlens[:-1].long(), normalize_output)
    if strategy in ("mean", "weighted_mean"):
        out = segment_mean(hidden, cu_seqlens, weighted=(strategy == "weighted_mean"))
        return normalize(out) if normalize_output else out
    raise ValueError(f"Unknown pooling strategy: {strategy}")
