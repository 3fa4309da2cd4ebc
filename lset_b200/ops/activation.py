"""SwiGLU / GeGLU gated activations and exact GELU.

``glu(gate_up, kind)`` takes the fused ``[T, 2I]`` projection output (gate columns first) and the
backward returns one ``[T, 2I]`` gradient, so a fused gate/up projection needs a single dgrad GEMM.
Counterparts: lset/kernels/swiglu.py:21-74, lset/kernels/geglu.py:22-86.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native as nv

_KINDS = {"swiglu": 0, "geglu": 1}


def glu_ref(gate, up, kind="swiglu"):
    if kind == "swiglu":
        return (F.silu(gate.float()) * up.float()).to(gate.dtype)
    return (F.gelu(gate.float(), approximate="tanh") * up.float()).to(gate.dtype)


class _GluFused(torch.autograd.Function):
    """gate_up: [T, 2I] contiguous."""

    @staticmethod
    def forward(ctx, gate_up, kind):
        T, I2 = gate_up.shape
        I = I2 // 2
        out = torch.empty(T, I, dtype=gate_up.dtype, device=gate_up.device)
        lib = nv.load()
        rc = lib.lb_glu_fwd(
            nv.c_int(kind), nv.c_void_p(gate_up.data_ptr()),
            nv.c_void_p(gate_up.data_ptr() + I * gate_up.element_size()), nv.c_ll(gate_up.stride(0)),
            nv.c_void_p(out.data_ptr()), nv.c_ll(I), nv.c_ll(T), nv.c_int(I),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_glu_fwd")
        nv.count_launch()
        ctx.save_for_backward(gate_up)
        ctx.kind = kind
        return out

    @staticmethod
    def backward(ctx, dout):
        (gate_up,) = ctx.saved_tensors
        T, I2 = gate_up.shape
        I = I2 // 2
        dout = dout if dout.is_contiguous() else dout.contiguous()
        dgu = torch.empty_like(gate_up)
        es = gate_up.element_size()
        lib = nv.load()
        rc = lib.lb_glu_bwd(
            nv.c_int(ctx.kind), nv.c_void_p(dout.data_ptr()), nv.c_ll(I),
            nv.c_void_p(gate_up.data_ptr()), nv.c_void_p(gate_up.data_ptr() + I * es),
            nv.c_ll(gate_up.stride(0)), nv.c_void_p(dgu.data_ptr()),
            nv.c_void_p(dgu.data_ptr() + I * es), nv.c_ll(I2), nv.c_ll(T), nv.c_int(I),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_glu_bwd")
        nv.count_launch()
        return dgu, None


def glu(gate_up, kind="swiglu"):
    """``act(gate) * up`` from the fused ``[..., 2I]`` tensor whose first half is the gate."""
    I = gate_up.shape[-1] // 2
    native = (nv.use_native(gate_up) and gate_up.dtype == torch.bfloat16 and I % 8 == 0)
    if not native:
        return glu_ref(gate_up[..., :I], gate_up[..., I:], kind)
    shape = gate_up.shape
    g2 = gate_up.reshape(-1, shape[-1])
    g2 = g2 if g2.is_contiguous() else g2.contiguous()
    return _GluFused.apply(g2, _KINDS[kind]).view(*shape[:-1], I)


def swiglu(gate, up):
    """``silu(gate) * up`` for separate gate / up tensors."""
    if not (nv.use_native(gate, up) and gate.dtype == torch.bfloat16 and gate.shape[-1] % 8 == 0):
        return glu_ref(gate, up, "swiglu")
    return glu(torch.cat([gate, up], dim=-1), "swiglu")


def geglu(gate, up):
    """``gelu_tanh(gate) * up`` for separate gate / up tensors."""
    if not (nv.use_native(gate, up) and gate.dtype == torch.bfloat16 and gate.shape[-1] % 8 == 0):
        return glu_ref(gate, up, "geglu")
    return glu(torch.cat([gate, up], dim=-1), "geglu")


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x if x.is_contiguous() else x.contiguous()
        y = torch.empty_like(xc)
        rc = nv.load().lb_gelu_fwd(nv.c_void_p(xc.data_ptr()), nv.c_void_p(y.data_ptr()),
                                   nv.c_ll(xc.numel()), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_gelu_fwd")
        nv.count_launch()
        ctx.save_for_backward(xc)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dx = torch.empty_like(x)
        rc = nv.load().lb_gelu_bwd(nv.c_void_p(dy.data_ptr()), nv.c_void_p(x.data_ptr()),
                                   nv.c_void_p(dx.data_ptr()), nv.c_ll(x.numel()),
                                   nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_gelu_bwd")
        nv.count_launch()
        return dx


def gelu(x):
    """Exact (erf) GELU."""
    if not (nv.use_native(x) and x.dtype == torch.bfloat16 and x.numel() % 8 == 0):
        return F.gelu(x)
    return _Gelu.apply(x)
