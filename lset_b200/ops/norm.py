"""RMSNorm / LayerNorm ops with optional fused residual add.

Every op has an eager PyTorch implementation (the numerics oracle, also the CPU path) and a native
sm_100a kernel behind an ``autograd.Function``. The eager code follows the rounding points of the
reference's kernels: statistics in fp32, the normalised value is cast to the input dtype before the
weight multiply, and the residual stream is stored in the activation dtype after an fp32 add
(lset/kernels/rmsnorm.py:68-73, lset/kernels/residual_rmsnorm.py:58-77,
lset/kernels/double_residual_rmsnorm.py:46-160, lset/kernels/layernorm.py:46-136,
lset/kernels/residual_layernorm.py:46-139).
"""
from __future__ import annotations

import torch

from . import _native as nv
from ._grads import main_grad_of
from .runtime_options import enabled


# --------------------------------------------------------------------------- eager oracles
def rms_norm_ref(x, w, eps=1e-6, w_off=0.0):
    if x.dtype == torch.float32 and not x.is_cuda and hasattr(torch.nn.functional, "rms_norm"):
        return torch.nn.functional.rms_norm(x, (x.shape[-1],), w + w_off if w_off else w, eps)
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wt = (w.float() + w_off).to(x.dtype) if w_off else w
    return (xf * rstd).to(x.dtype) * wt.to(x.dtype)


def residual_rms_norm_ref(residual, x, w, eps=1e-6, w_off=0.0):
    nr = (residual.float() + x.float()).to(x.dtype)
    return rms_norm_ref(nr, w, eps, w_off), nr


def layer_norm_ref(x, w, b, eps=1e-12):
    if x.dtype == torch.float32 and not x.is_cuda:
        # CPU fp32 training path: the library's fused kernel computes the same thing (there are no
        # intermediate roundings to reproduce in fp32) several times faster than the explicit form
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), w, b, eps)
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).pow(2).mean(-1, keepdim=True)
    y = ((xf - mean) * torch.rsqrt(var + eps)).to(x.dtype) * w.to(x.dtype)
    return y + b.to(x.dtype) if b is not None else y


def residual_layer_norm_ref(residual, x, w, b, eps=1e-12):
    nr = (residual.float() + x.float()).to(x.dtype)
    return layer_norm_ref(nr, w, b, eps), nr


def double_residual_rms_norm_ref(residual, a, w1, w2, eps=1e-6, w_off=0.0):
    z = rms_norm_ref(a, w1, eps, w_off)
    nr = (residual.float() + z.float()).to(a.dtype)
    return rms_norm_ref(nr, w2, eps, w_off), nr


# --------------------------------------------------------------------------- helpers
_scratch = {}


def scratch(name: str, numel: int, device) -> torch.Tensor:
    """Reusable fp32 scratch buffer (per name and device), grown on demand."""
    key = (name, device.index)
    t = _scratch.get(key)
    if t is None or t.numel() < numel:
        t = torch.empty(numel, dtype=torch.float32, device=device)
        _scratch[key] = t
    return t


def _native_ok(*ts):
    return nv.use_native(*ts) and all(t is None or t.dtype == torch.bfloat16 for t in ts)


def deliver_wgrad(w, n_values: int, device, kernel_call):
    """Run ``kernel_call(out_ptr, out_is_fp32, accumulate)`` so that the weight gradient lands either
    in ``w.main_grad`` (fp32 accumulator owned by the sharding runtime; returns None) or in a fresh
    tensor of ``w``'s dtype (returned)."""
    main = main_grad_of(w)
    if main is not None:
        kernel_call(main.data_ptr(), 1, 1)
        return None
    out = torch.empty(n_values, dtype=torch.float32, device=device)
    kernel_call(out.data_ptr(), 1, 0)
    return out


# --------------------------------------------------------------------------- RMSNorm
class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps, w_off):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        N = x2.shape[0]
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
        y = torch.empty_like(x2)
        res_out = torch.empty_like(x2) if r2 is not None else None
        rstd = torch.empty(N, dtype=torch.float32, device=x.device)
        lib = nv.load()
        rc = lib.lb_rms_norm_fwd(
            nv.c_void_p(x2.data_ptr()), nv.c_void_p(nv.ptr(r2)), nv.c_void_p(w.data_ptr()),
            nv.c_void_p(y.data_ptr()), nv.c_void_p(nv.ptr(res_out)), nv.c_void_p(rstd.data_ptr()),
            nv.c_int(N), nv.c_int(H), nv.c_float(eps), nv.c_float(w_off),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_rms_norm_fwd")
        nv.count_launch()
        ctx.save_for_backward(res_out if r2 is not None else x2, w, rstd)
        ctx.w_off = w_off
        ctx.has_res = r2 is not None
        ctx.shape = shape
        if r2 is not None:
            return y.view(shape), res_out.view(shape)
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, dres):
        xin, w, rstd = ctx.saved_tensors
        dx, dw = _rms_bwd(dy, dres if ctx.has_res else None, xin, w, rstd, ctx.w_off,
                          ctx.needs_input_grad[2])
        dxv = dx.view(ctx.shape)
        return dxv, (dxv if ctx.has_res else None), dw, None, None


def _rms_bwd(dy, dres, xin, w, rstd, w_off, need_dw):
    """One RMSNorm backward launch: ``dx`` (plus ``dres`` when given) and the weight gradient,
    which lands in ``w.main_grad`` when the sharding runtime provides one (then ``dw`` is None)."""
    N, H = xin.shape
    dy2 = dy.reshape(N, H)
    dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
    dr2 = None
    if dres is not None:
        dr2 = dres.reshape(N, H)
        dr2 = dr2 if dr2.is_contiguous() else dr2.contiguous()
    dx = torch.empty_like(xin)
    lib = nv.load()
    rows = lib.lb_norm_bwd_partial_rows()
    scr = scratch("norm_bwd", rows * H, xin.device)

    def call(out_ptr, out_fp32, accumulate):
        rc = lib.lb_rms_norm_bwd(
            nv.c_void_p(dy2.data_ptr()), nv.c_void_p(nv.ptr(dr2)), nv.c_void_p(xin.data_ptr()),
            nv.c_void_p(w.data_ptr()), nv.c_void_p(rstd.data_ptr()), nv.c_void_p(dx.data_ptr()),
            nv.c_void_p(scr.data_ptr()), nv.c_void_p(out_ptr), nv.c_int(out_fp32),
            nv.c_int(accumulate), nv.c_int(N), nv.c_int(H), nv.c_float(w_off),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_rms_norm_bwd")
        nv.count_launch(2 if out_ptr else 1)

    dw = None
    if need_dw:
        dw = deliver_wgrad(w, H, xin.device, call)
        if dw is not None:
            dw = dw.to(w.dtype)
    else:
        call(0, 1, 0)
    return dx, dw


class _RmsNormDouble(torch.autograd.Function):
    """``z = rmsnorm(a)·w1; nr = residual + z; y = rmsnorm(nr)·w2`` in one forward launch; the
    backward is the two single-norm launches."""

    @staticmethod
    def forward(ctx, residual, a, w1, w2, eps, w_off):
        shape = a.shape
        H = shape[-1]
        a2 = a.reshape(-1, H)
        a2 = a2 if a2.is_contiguous() else a2.contiguous()
        r2 = residual.reshape(-1, H)
        r2 = r2 if r2.is_contiguous() else r2.contiguous()
        N = a2.shape[0]
        y, nr = torch.empty_like(a2), torch.empty_like(a2)
        rstd1 = torch.empty(N, dtype=torch.float32, device=a.device)
        rstd2 = torch.empty(N, dtype=torch.float32, device=a.device)
        rc = nv.load().lb_rms_norm_double_fwd(
            nv.c_void_p(a2.data_ptr()), nv.c_void_p(r2.data_ptr()), nv.c_void_p(w1.data_ptr()),
            nv.c_void_p(w2.data_ptr()), nv.c_void_p(y.data_ptr()), nv.c_void_p(nr.data_ptr()),
            nv.c_void_p(rstd1.data_ptr()), nv.c_void_p(rstd2.data_ptr()), nv.c_int(N), nv.c_int(H),
            nv.c_float(eps), nv.c_float(w_off), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_rms_norm_double_fwd")
        nv.count_launch()
        ctx.save_for_backward(a2, nr, w1, w2, rstd1, rstd2)
        ctx.w_off, ctx.shape = w_off, shape
        return y.view(shape), nr.view(shape)

    @staticmethod
    def backward(ctx, dy, dnr):
        a2, nr, w1, w2, rstd1, rstd2 = ctx.saved_tensors
        d_nr, dw2 = _rms_bwd(dy, dnr, nr, w2, rstd2, ctx.w_off, ctx.needs_input_grad[3])
        d_a, dw1 = _rms_bwd(d_nr, None, a2, w1, rstd1, ctx.w_off, ctx.needs_input_grad[2])
        return d_nr.view(ctx.shape), d_a.view(ctx.shape), dw1, dw2, None, None


def rms_norm(x, w, eps=1e-6, w_off=0.0):
    """``y = bf16(x * rsqrt(mean(x²) + eps)) * (w + w_off)``."""
    if not (_native_ok(x, w) and enabled("fused_rmsnorm")):
        return rms_norm_ref(x, w, eps, w_off)
    return _RmsNorm.apply(x, None, w, eps, w_off)[0]


def residual_rms_norm(residual, x, w, eps=1e-6, w_off=0.0):
    """``nr = residual + x`` then RMSNorm; returns ``(y, nr)``."""
    if not (_native_ok(residual, x, w) and enabled("fused_residual_rmsnorm")):
        return residual_rms_norm_ref(residual, x, w, eps, w_off)
    return _RmsNorm.apply(x, residual, w, eps, w_off)


def double_residual_rms_norm(residual, a, w1, w2, eps=1e-6, w_off=0.0):
    """Gemma post-norm pair: ``z = rmsnorm(a)·w1; nr = residual + z; out = rmsnorm(nr)·w2``;
    returns ``(out, nr)``. One forward launch (the row never leaves the registers between the two
    norms); rows wider than 6144 take the two-launch route."""
    if not (_native_ok(residual, a, w1, w2) and enabled("fused_double_rmsnorm")):
        return double_residual_rms_norm_ref(residual, a, w1, w2, eps, w_off)
    if a.shape[-1] * 8 > 48 * 1024:
        z = rms_norm(a, w1, eps, w_off)
        return residual_rms_norm(residual, z, w2, eps, w_off)
    return _RmsNormDouble.apply(residual, a, w1, w2, eps, w_off)


# --------------------------------------------------------------------------- LayerNorm
class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, b, eps):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        N = x2.shape[0]
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
        y = torch.empty_like(x2)
        res_out = torch.empty_like(x2) if r2 is not None else None
        mean = torch.empty(N, dtype=torch.float32, device=x.device)
        rstd = torch.empty(N, dtype=torch.float32, device=x.device)
        lib = nv.load()
        rc = lib.lb_layer_norm_fwd(
            nv.c_void_p(x2.data_ptr()), nv.c_void_p(nv.ptr(r2)), nv.c_void_p(w.data_ptr()),
            nv.c_void_p(nv.ptr(b)), nv.c_void_p(y.data_ptr()), nv.c_void_p(nv.ptr(res_out)),
            nv.c_void_p(mean.data_ptr()), nv.c_void_p(rstd.data_ptr()), nv.c_int(N), nv.c_int(H),
            nv.c_float(eps), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_layer_norm_fwd")
        nv.count_launch()
        ctx.save_for_backward(res_out if r2 is not None else x2, w, mean, rstd)
        ctx.has_res = r2 is not None
        ctx.has_bias = b is not None
        ctx.b_ref = b
        ctx.shape = shape
        return y.view(shape), (res_out.view(shape) if r2 is not None else None)

    @staticmethod
    def backward(ctx, dy, dres):
        xin, w, mean, rstd = ctx.saved_tensors
        N, H = xin.shape
        dy2 = dy.reshape(N, H)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dr2 = None
        if dres is not None and ctx.has_res:
            dr2 = dres.reshape(N, H)
            dr2 = dr2 if dr2.is_contiguous() else dr2.contiguous()
        dx = torch.empty_like(xin)
        lib = nv.load()
        rows = lib.lb_norm_bwd_partial_rows()
        scr = scratch("norm_bwd", rows * 2 * H, xin.device)
        dwb = torch.empty(2 * H, dtype=torch.float32, device=xin.device)
        rc = lib.lb_layer_norm_bwd(
            nv.c_void_p(dy2.data_ptr()), nv.c_void_p(nv.ptr(dr2)), nv.c_void_p(xin.data_ptr()),
            nv.c_void_p(w.data_ptr()), nv.c_void_p(mean.data_ptr()), nv.c_void_p(rstd.data_ptr()),
            nv.c_void_p(dx.data_ptr()), nv.c_void_p(scr.data_ptr()), nv.c_void_p(dwb.data_ptr()),
            nv.c_int(1), nv.c_int(0), nv.c_int(N), nv.c_int(H), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_layer_norm_bwd")
        nv.count_launch(2)
        dw = db = None
        b = ctx.b_ref
        mg = main_grad_of(w)
        if mg is not None:
            mg.add_(dwb[:H])
        else:
            dw = dwb[:H].to(w.dtype)
        if ctx.has_bias:
            mgb = main_grad_of(b)
            if mgb is not None:
                mgb.add_(dwb[H:])
            else:
                db = dwb[H:].to(b.dtype)
        dxv = dx.view(ctx.shape)
        return dxv, (dxv if ctx.has_res else None), dw, db, None


def layer_norm(x, w, b, eps=1e-12):
    if not (_native_ok(x, w, b) and enabled("fused_layernorm")):
        return layer_norm_ref(x, w, b, eps)
    return _LayerNorm.apply(x, None, w, b, eps)[0]


def residual_layer_norm(residual, x, w, b, eps=1e-12):
    """``nr = residual + x`` then LayerNorm; returns ``(y, nr)`` (BERT post-norm)."""
    if not (_native_ok(residual, x, w, b) and enabled("fused_layernorm")):
        return residual_layer_norm_ref(residual, x, w, b, eps)
    return _LayerNorm.apply(x, residual, w, b, eps)
