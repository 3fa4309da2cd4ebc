"""bf16 GEMM on the tcgen05 kernel, and the ``linear`` autograd op built from its three forms.

``matmul_abt`` computes ``C = A · Bᵀ`` where each operand is either K-major (``[rows, K]``, the
layout of activations and ``nn.Linear`` weights) or MN-major (``[K, rows]``). The backward of a
linear layer uses the MN-major forms so no tensor is ever transposed in memory.

Replaces the cuBLAS calls behind ``nn.Linear`` in the reference
(lset/models/decoder/qwen3/attention.py:102-104, lset/models/decoder/qwen3/mlp.py:28).
"""
from __future__ import annotations


import torch

from . import _native as nv
from ._grads import main_grad_of
from ._ac import run_expensive


def _oracle(a, b, a_mn, b_mn, bias, out_dtype):
    af = a.float().t() if a_mn else a.float()
    bf = b.float().t() if b_mn else b.float()
    c = af @ bf.t()
    if bias is not None:
        c = c + bias.float()
    return c.to(out_dtype)


def matmul_abt(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=torch.bfloat16,
               accumulate=False, bias=None, splits=1, bn=0):
    """``C[M,N] = A · Bᵀ`` with fp32 accumulation.

    a: ``[M, K]`` (``[K, M]`` when ``a_mn``), b: ``[N, K]`` (``[K, N]`` when ``b_mn``); 2-D bf16
    with unit inner stride. ``out`` may be given (fp32 with ``accumulate=True`` adds into it).
    ``splits > 1`` splits the contraction and reduces with fp32 atomics (fp32 output only);
    ``splits=0`` lets the launcher choose the split from the tile count and the contraction length.
    """
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("matmul_abt takes 2-D operands")
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    if K != Kb:
        raise ValueError(f"contraction mismatch: {K} vs {Kb}")
    if out is not None:
        out_dtype = out.dtype
    if not nv.use_native(a, b):
        c = _oracle(a, b, a_mn, b_mn, bias, torch.float32 if accumulate else out_dtype)
        if out is not None:
            if accumulate:
                out.add_(c.to(out.dtype))
            else:
                out.copy_(c)
            return out
        return c
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("matmul_abt runs bf16 operands on the GPU")
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("output must be bf16 or fp32")
    if splits != 1 and out_dtype != torch.float32:
        splits = 1
    auto = splits == 0
    if out is None:
        if accumulate or splits != 1:
            out = torch.zeros(M, N, dtype=out_dtype, device=a.device)
        else:
            out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    elif splits != 1 and not accumulate:
        out.zero_()
    if M == 0 or N == 0:
        return out
    if K == 0:
        if not accumulate:
            out.zero_()
        return out
    if bias is not None and bias.dtype != torch.bfloat16:
        bias = bias.to(torch.bfloat16)
    lib = nv.load()
    rc = lib.lb_gemm_bf16(
        nv.c_void_p(a.data_ptr()), nv.c_void_p(b.data_ptr()), nv.c_void_p(out.data_ptr()),
        nv.c_int(M), nv.c_int(N), nv.c_int(K),
        nv.c_ll(a.stride(0)), nv.c_ll(b.stride(0)), nv.c_ll(out.stride(0)),
        nv.c_int(int(a_mn)), nv.c_int(int(b_mn)), nv.c_int(int(out_dtype == torch.float32)),
        nv.c_int(int(accumulate or splits > 1 or auto)), nv.c_void_p(nv.ptr(bias)), nv.c_int(splits),
        nv.c_int(bn), nv.c_void_p(nv.status_word(a.device).data_ptr()),
        nv.c_void_p(nv.stream_ptr()),
    )
    if rc != 0:
        nv.check_rc(rc, f"lb_gemm_bf16(M={M},N={N},K={K})")
    nv.count_launch()
    return out


def wgrad_splits(n_out: int, k_in: int, tokens: int) -> int:
    """Split of the token contraction of a ``[n_out, k_in]`` weight gradient: 0 = chosen by the
    launcher (``auto_splits`` in csrc/gemm/gemm_bf16.cu: whole waves of work items over the SMs,
    items long enough to hide their reduction epilogue)."""
    return 0


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        y = run_expensive(lambda: matmul_abt(x2, w, bias=bias))
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16 and dy2.is_cuda:
            dy2 = dy2.to(torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = matmul_abt(dy2, w, b_mn=True).view_as(x)
        if ctx.needs_input_grad[1]:
            main = main_grad_of(w)
            if main is not None and dy2.is_cuda:
                # fp32 gradient accumulator owned by the sharding runtime: add straight into it.
                matmul_abt(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True,
                           splits=wgrad_splits(w.shape[0], w.shape[1], x2.shape[0]))
                dw = None
            else:
                dw = matmul_abt(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32,
                                splits=wgrad_splits(w.shape[0], w.shape[1], x2.shape[0])
                                if dy2.is_cuda else 1).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x, w, bias=None):
    """``y = x · wᵀ (+ bias)`` — drop-in for ``F.linear`` on bf16 CUDA tensors; eager on CPU/fp32."""
    if not nv.use_native(x, w) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return torch.nn.functional.linear(x, w, bias)
    return _Linear.apply(x, w, bias)


def matmul_ext(a, b, a2, b2, *, b_mn=False, bias=None):
    """``A · op(B) + A2 · op(B2)`` (bf16 out) in one pass over the accumulator: the second pair's
    k-blocks are appended to the contraction (``lb_gemm_bf16_ext``). ``op`` as in ``matmul_abt``;
    ``a2`` is ``[M, K2]`` with K2 a multiple of 8 (a LoRA rank)."""
    M, K = a.shape
    K2 = a2.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    if not nv.use_native(a, b, a2, b2):
        bf = b.float() if b_mn else b.float().t()
        b2f = b2.float() if b_mn else b2.float().t()
        c = a.float() @ bf + a2.float() @ b2f
        if bias is not None:
            c = c + bias.float()
        return c.to(a.dtype)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    if M == 0 or N == 0:
        return out
    rc = nv.load().lb_gemm_bf16_ext(
        nv.c_void_p(a.data_ptr()), nv.c_void_p(b.data_ptr()), nv.c_void_p(a2.data_ptr()),
        nv.c_void_p(b2.data_ptr()), nv.c_void_p(out.data_ptr()), nv.c_int(M), nv.c_int(N),
        nv.c_int(K), nv.c_int(K2), nv.c_ll(a.stride(0)), nv.c_ll(b.stride(0)),
        nv.c_ll(a2.stride(0)), nv.c_ll(b2.stride(0)), nv.c_ll(N), nv.c_int(int(b_mn)),
        nv.c_void_p(nv.ptr(bias)), nv.c_void_p(nv.status_word(a.device).data_ptr()),
        nv.c_void_p(nv.stream_ptr()))
    if rc != 0:
        nv.check_rc(rc, f"lb_gemm_bf16_ext(M={M},N={N},K={K},K2={K2})")
    nv.count_launch()
    return out


def _accumulate_wgrad(w, dy2, x2):
    """``dW = dy2ᵀ · x2`` into ``w.main_grad`` (returns None) or as a tensor of ``w``'s dtype."""
    splits = wgrad_splits(w.shape[0], w.shape[1], x2.shape[0]) if dy2.is_cuda else 1
    main = main_grad_of(w)
    if main is not None and dy2.is_cuda:
        matmul_abt(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True, splits=splits)
        return None
    return matmul_abt(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32,
                      splits=splits).to(w.dtype)


class _LoRALinear(torch.autograd.Function):
    """``y = x Wᵀ + s · (x Aᵀ) Bᵀ (+ bias)`` with a frozen ``W``: the rank-r update rides along in
    the base GEMM's accumulator (forward) and in the input-gradient GEMM (backward), so the
    ``[T, N]`` output is written once and never re-read. No weight gradient for ``W``."""

    @staticmethod
    def forward(ctx, x, w, lora_a, lora_b, bias, scale):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        t = matmul_abt(x2, lora_a)                       # [T, r]
        ts = t * scale
        # kept across selective activation checkpointing like every other big GEMM output
        y = run_expensive(lambda: matmul_ext(x2, w, ts, lora_b, bias=bias))   # x·Wᵀ + ts·Bᵀ
        ctx.save_for_backward(x2, ts, w, lora_a, lora_b)
        ctx.scale = scale
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, ts, w, lora_a, lora_b = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16 and dy2.is_cuda:
            dy2 = dy2.to(torch.bfloat16)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        us = matmul_abt(dy2, lora_b, b_mn=True) * ctx.scale          # [T, r] = s · dy · B
        dx = None
        if ctx.needs_input_grad[0]:
            dx = matmul_ext(dy2, w, us, lora_a, b_mn=True).view(ctx.shape)   # dy·W + us·A
        da = _accumulate_wgrad(lora_a, us, x2) if ctx.needs_input_grad[2] else None   # usᵀ · x
        db = _accumulate_wgrad(lora_b, dy2, ts) if ctx.needs_input_grad[3] else None  # dyᵀ · ts
        dbias = dy2.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[4] else None
        return dx, None, da, db, dbias, None


def lora_linear(x, w, lora_a, lora_b, bias, scale: float):
    return _LoRALinear.apply(x, w, lora_a, lora_b, bias, float(scale))


_GLU_KINDS = {"swiglu": 0, "geglu": 1}


class _LinearGlu(torch.autograd.Function):
    """``h = act(x·Wgᵀ) * (x·Wuᵀ)`` for the fused weight ``W = [Wg; Wu]``: the activation runs in
    the GEMM epilogue (``lb_gemm_glu``), so the ``[T, 2I]`` projection output is written once (for
    the backward) and never read back in the forward."""

    @staticmethod
    def forward(ctx, x, w, kind):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        T, K = x2.shape
        I = w.shape[0] // 2

        def launch():
            gu = torch.empty(T, 2 * I, dtype=torch.bfloat16, device=x.device)
            h = torch.empty(T, I, dtype=torch.bfloat16, device=x.device)
            rc = nv.load().lb_gemm_glu(
                nv.c_void_p(x2.data_ptr()), nv.c_void_p(w.data_ptr()), nv.c_void_p(gu.data_ptr()),
                nv.c_void_p(h.data_ptr()), nv.c_int(T), nv.c_int(I), nv.c_int(K), nv.c_ll(K),
                nv.c_ll(w.stride(0)), nv.c_ll(2 * I), nv.c_ll(I), nv.c_int(kind),
                nv.c_void_p(nv.status_word(x.device).data_ptr()), nv.c_void_p(nv.stream_ptr()))
            if rc != 0:
                nv.check_rc(rc, f"lb_gemm_glu(T={T},I={I},K={K})")
            nv.count_launch()
            return h, gu

        h, gu = run_expensive(launch)
        ctx.save_for_backward(x2, w, gu)
        ctx.kind = kind
        ctx.shape = x.shape
        return h.view(*x.shape[:-1], I)

    @staticmethod
    def backward(ctx, dh):
        x2, w, gu = ctx.saved_tensors
        T, I2 = gu.shape
        I = I2 // 2
        dh2 = dh.reshape(T, I)
        dh2 = dh2 if dh2.is_contiguous() else dh2.contiguous()
        dgu = torch.empty_like(gu)
        rc = nv.load().lb_glu_bwd(
            nv.c_int(ctx.kind), nv.c_void_p(dh2.data_ptr()), nv.c_ll(I),
            nv.c_void_p(gu.data_ptr()), nv.c_void_p(gu.data_ptr() + 2 * I), nv.c_ll(I2),
            nv.c_void_p(dgu.data_ptr()), nv.c_void_p(dgu.data_ptr() + 2 * I), nv.c_ll(I2),
            nv.c_ll(T), nv.c_int(I), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_glu_bwd")
        nv.count_launch()
        dx = matmul_abt(dgu, w, b_mn=True).view(ctx.shape) if ctx.needs_input_grad[0] else None
        dw = _accumulate_wgrad(w, dgu, x2) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def linear_glu_supported(x, w) -> bool:
    return (nv.use_native(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[0] % 16 == 0 and x.shape[-1] % 8 == 0 and w.stride(1) == 1)


def linear_glu(x, w, kind: str = "swiglu"):
    """Gated-MLP input projection + activation; ``w`` is the fused ``[2I, K]`` gate/up weight."""
    return _LinearGlu.apply(x, w, _GLU_KINDS[kind])
