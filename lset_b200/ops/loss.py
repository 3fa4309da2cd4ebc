"""Similarity product for the contrastive losses.

``similarity(q, k)`` returns the fp32 score matrix ``q · kᵀ``. For bf16 CUDA inputs the forward and
both gradient products run on the tcgen05 GEMM (no transposes: the passage-gradient product
consumes the score gradient and the queries as MN-major operands); elsewhere it is a plain matmul.
Replaces the cuBLAS matmul of lset/losses/infonce.py:20 and lset/losses/contrastive.py:22.
"""
from __future__ import annotations

import torch

from . import _native as nv
from .gemm import matmul_abt


class _Similarity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k):
        ctx.save_for_backward(q, k)
        return matmul_abt(q, k, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, ds):
        q, k = ctx.saved_tensors
        Q, K = ds.shape
        # bf16 copy of the score gradient with a row stride that is a multiple of 8 elements
        Kp = (K + 7) // 8 * 8
        Qp = (Q + 7) // 8 * 8
        g = torch.zeros(Qp, Kp, dtype=torch.bfloat16, device=ds.device)
        g[:Q, :K] = ds
        dq = dk = None
        if ctx.needs_input_grad[0]:
            kp = k if Kp == K else torch.cat([k, k.new_zeros(Kp - K, k.shape[1])])
            dq = matmul_abt(g[:Q], kp, b_mn=True)                     # [Q, D] = g · k
        if ctx.needs_input_grad[1]:
            qp = q if Qp == Q else torch.cat([q, q.new_zeros(Qp - Q, q.shape[1])])
            dk = matmul_abt(g, qp, a_mn=True, b_mn=True)[:K]          # [K, D] = gᵀ · q
        return dq, dk


def similarity(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """fp32 ``[Q, K]`` scores of ``q [Q, D]`` against ``k [K, D]``."""
    native = (nv.use_native(q, k) and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
              and q.shape[1] % 8 == 0 and k.shape[0] % 8 == 0)
    if native:
        return _Similarity.apply(q.contiguous(), k.contiguous())
    return q.float() @ k.float().t()


# ------------------------------------------------------------------------------------------------
# Streaming InfoNCE: scores never materialise in fp32; see lb_infonce_fwd / lb_infonce_pgrad.
# ------------------------------------------------------------------------------------------------
class _FusedInfoNCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, inv_t, target_offset, denom):
        M, D = q.shape
        N = k.shape[0]
        lib = nv.load()
        lib.lb_infonce_scratch_floats.restype = nv.c_ll
        scr = torch.empty(int(lib.lb_infonce_scratch_floats(nv.c_int(M), nv.c_int(N))),
                          dtype=torch.float32, device=q.device)
        lse = torch.empty(M, dtype=torch.float32, device=q.device)
        loss_sum = torch.zeros(1, dtype=torch.float32, device=q.device)
        rc = lib.lb_infonce_fwd(
            nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), nv.c_void_p(k.data_ptr()),
            nv.c_ll(k.stride(0)), nv.c_int(M), nv.c_int(N), nv.c_int(D), nv.c_float(inv_t),
            nv.c_ll(target_offset), nv.c_void_p(scr.data_ptr()), nv.c_void_p(lse.data_ptr()),
            nv.c_void_p(loss_sum.data_ptr()), nv.c_void_p(nv.status_word(q.device).data_ptr()),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_infonce_fwd")
        nv.count_launch(2)
        ctx.save_for_backward(q, k, lse)
        ctx.meta = (inv_t, target_offset, denom)
        return loss_sum[0] / denom

    @staticmethod
    def backward(ctx, g):
        q, k, lse = ctx.saved_tensors
        inv_t, target_offset, denom = ctx.meta
        M, D = q.shape
        N = k.shape[0]
        coef = (g.float() * (inv_t / denom)).reshape(1).contiguous()
        Mp = (M + 7) // 8 * 8
        W = torch.empty(Mp, N, dtype=torch.bfloat16, device=q.device)
        if Mp != M:
            W[M:].zero_()
        rc = nv.load().lb_infonce_pgrad(
            nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), nv.c_void_p(k.data_ptr()),
            nv.c_ll(k.stride(0)), nv.c_int(M), nv.c_int(N), nv.c_int(D), nv.c_float(inv_t),
            nv.c_ll(target_offset), nv.c_void_p(lse.data_ptr()), nv.c_void_p(coef.data_ptr()),
            nv.c_void_p(W.data_ptr()), nv.c_ll(N), nv.c_void_p(nv.status_word(q.device).data_ptr()),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_infonce_pgrad")
        nv.count_launch()
        dq = dk = None
        if ctx.needs_input_grad[0]:
            dq = matmul_abt(W[:M], k, b_mn=True)                                # [M, D] = W · K
        if ctx.needs_input_grad[1]:
            qp = q if Mp == M else torch.cat([q, q.new_zeros(Mp - M, D)])
            dk = matmul_abt(W, qp, a_mn=True, b_mn=True)                        # [N, D] = Wᵀ · Q
        return dq, dk, None, None, None


def fused_infonce_supported(q, k) -> bool:
    return (nv.use_native(q, k) and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
            and q.shape[1] % 8 == 0 and k.shape[0] % 8 == 0 and q.shape[1] == k.shape[1])


def fused_infonce(q, k, temperature: float, target_offset: int = 0, denom: float | None = None):
    """``sum_r CE(q_r · Kᵀ / T, r + target_offset) / denom`` (``denom`` defaults to the number of
    queries) on the streaming tcgen05 kernels. ``temperature`` must be a Python float."""
    denom = float(denom if denom is not None else q.shape[0])
    return _FusedInfoNCE.apply(q.contiguous(), k.contiguous(), 1.0 / float(temperature),
                               int(target_offset), denom)
