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
