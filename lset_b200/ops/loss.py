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
# Backward of the streaming losses in column panels.
#
# The probability gradient W = (softmax - target) * coef is needed as a bf16 operand of two more
# products (dQ = W · K, dK = Wᵀ · Q). It is never held as a whole [Q, K] matrix: the passages are
# walked in panels of columns, the panel's W is recomputed from the saved row LSE, dK of the panel
# is complete after one product, and dQ accumulates over the panels in fp32. A panel's W is capped
# at PANEL_BYTES (half of the 126 MB L2, so the two products that read it find it there); score
# matrices below the cap take a single panel. Extra memory: the cap plus the fp32 accumulator of dQ.
# ------------------------------------------------------------------------------------------------
PANEL_BYTES = 64 << 20
PANEL_MIN_COLS = 1024       # narrower panels leave the dK product too few tiles


def panel_cols(M: int, N: int) -> int:
    """Columns per panel for M query rows: as many as fit PANEL_BYTES of bf16, a multiple of 256
    (the loss kernels' column tile; keeps label rows 16-byte aligned), at least PANEL_MIN_COLS."""
    Mp = (M + 7) // 8 * 8
    cols = max(PANEL_MIN_COLS, (PANEL_BYTES // (2 * Mp)) // 256 * 256)
    return min(N, cols)


def streamed_loss_backward(launch_pgrad, q, k, need_dq: bool, need_dk: bool):
    """``launch_pgrad(c0, c1, W)`` fills ``W [Mp, c1 - c0]`` (bf16, rows past M zero) for the
    passage columns ``[c0, c1)``. Returns ``(dq, dk)`` in the inputs' dtype."""
    M, D = q.shape
    N = k.shape[0]
    Mp = (M + 7) // 8 * 8
    step = panel_cols(M, N)
    single = step >= N
    qp = q if Mp == M else torch.cat([q, q.new_zeros(Mp - M, D)])
    dq = dk = dq32 = None
    if need_dk:
        dk = torch.empty(N, D, dtype=k.dtype, device=k.device)
    W = torch.empty(Mp, step, dtype=torch.bfloat16, device=q.device)
    if Mp != M:
        W[M:].zero_()
    for c0 in range(0, N, step):
        c1 = min(N, c0 + step)
        Wp = W if c1 - c0 == step else W[:, :c1 - c0]
        launch_pgrad(c0, c1, Wp)
        if need_dq:
            if single:
                dq = matmul_abt(Wp[:M], k, b_mn=True)                       # [M, D] = W · K
            elif dq32 is None:
                dq32 = matmul_abt(Wp[:M], k[c0:c1], b_mn=True, out_dtype=torch.float32)
            else:
                matmul_abt(Wp[:M], k[c0:c1], b_mn=True, out=dq32, accumulate=True)
        if need_dk:
            matmul_abt(Wp, qp, a_mn=True, b_mn=True, out=dk[c0:c1])         # [n, D] = Wᵀ · Q
    if need_dq and dq is None:
        dq = dq32.to(q.dtype)
    return dq, dk


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
        lib = nv.load()
        status = nv.status_word(q.device).data_ptr()

        def pgrad(c0, c1, W):
            # columns [c0, c1): the passages start at row c0, the target column moves by -c0
            rc = lib.lb_infonce_pgrad(
                nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)),
                nv.c_void_p(k.data_ptr() + c0 * k.stride(0) * k.element_size()),
                nv.c_ll(k.stride(0)), nv.c_int(M), nv.c_int(c1 - c0), nv.c_int(D), nv.c_float(inv_t),
                nv.c_ll(target_offset - c0), nv.c_void_p(lse.data_ptr()),
                nv.c_void_p(coef.data_ptr()), nv.c_void_p(W.data_ptr()), nv.c_ll(W.stride(0)),
                nv.c_void_p(status), nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_infonce_pgrad")
            nv.count_launch()

        dq, dk = streamed_loss_backward(pgrad, q, k, ctx.needs_input_grad[0],
                                        ctx.needs_input_grad[1])
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


# ------------------------------------------------------------------------------------------------
# Streaming label-matrix loss (multi-positive NCE / soft-label cross-entropy): the [Q, K] scores
# exist only as tensor-core accumulators; see lb_label_loss_fwd / lb_label_loss_pgrad.
# ------------------------------------------------------------------------------------------------
class _FusedLabelLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, labels8, tw, row_scale, row_w, inv_t):
        M, D = q.shape
        N = k.shape[0]
        lib = nv.load()
        lib.lb_infonce_scratch_floats.restype = nv.c_ll
        scr = torch.empty(int(lib.lb_infonce_scratch_floats(nv.c_int(M), nv.c_int(N))),
                          dtype=torch.float32, device=q.device)
        lse = torch.empty(M, dtype=torch.float32, device=q.device)
        loss_sum = torch.zeros(1, dtype=torch.float32, device=q.device)
        rc = lib.lb_label_loss_fwd(
            nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), nv.c_void_p(k.data_ptr()),
            nv.c_ll(k.stride(0)), nv.c_int(M), nv.c_int(N), nv.c_int(D), nv.c_float(inv_t),
            nv.c_void_p(labels8.data_ptr()), nv.c_ll(labels8.stride(0)),
            nv.c_void_p(tw.data_ptr() if tw is not None else None),
            nv.c_ll(tw.stride(0) if tw is not None else 0), nv.c_void_p(row_scale.data_ptr()),
            nv.c_void_p(row_w.data_ptr()), nv.c_int(0), nv.c_void_p(scr.data_ptr()),
            nv.c_void_p(lse.data_ptr()),
            nv.c_void_p(loss_sum.data_ptr()), nv.c_void_p(nv.status_word(q.device).data_ptr()),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_label_loss_fwd")
        nv.count_launch(2)
        ctx.save_for_backward(q, k, lse, labels8, row_scale, row_w, *([tw] if tw is not None else []))
        ctx.inv_t = inv_t
        return loss_sum[0]

    @staticmethod
    def backward(ctx, g):
        q, k, lse, labels8, row_scale, row_w, *rest = ctx.saved_tensors
        tw = rest[0] if rest else None
        inv_t = ctx.inv_t
        M, D = q.shape
        N = k.shape[0]
        coef = (g.float() * inv_t).reshape(1).contiguous()
        lib = nv.load()
        status = nv.status_word(q.device).data_ptr()

        def pgrad(c0, c1, W):
            # panel starts are multiples of 256 columns: the int8 label rows stay 16-byte aligned
            rc = lib.lb_label_loss_pgrad(
                nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)),
                nv.c_void_p(k.data_ptr() + c0 * k.stride(0) * k.element_size()),
                nv.c_ll(k.stride(0)), nv.c_int(M), nv.c_int(c1 - c0), nv.c_int(D), nv.c_float(inv_t),
                nv.c_void_p(labels8.data_ptr() + c0), nv.c_ll(labels8.stride(0)),
                nv.c_void_p(tw.data_ptr() + 4 * c0 if tw is not None else None),
                nv.c_ll(tw.stride(0) if tw is not None else 0), nv.c_void_p(row_scale.data_ptr()),
                nv.c_void_p(row_w.data_ptr()), nv.c_int(0), nv.c_void_p(lse.data_ptr()),
                nv.c_void_p(coef.data_ptr()), nv.c_void_p(W.data_ptr()), nv.c_ll(W.stride(0)),
                nv.c_void_p(status), nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_label_loss_pgrad")
            nv.count_launch()

        dq, dk = streamed_loss_backward(pgrad, q, k, ctx.needs_input_grad[0],
                                        ctx.needs_input_grad[1])
        return dq, dk, None, None, None, None, None


def fused_label_loss_supported(q, k) -> bool:
    return (nv.use_native(q, k) and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
            and q.shape[1] % 8 == 0 and q.shape[1] == k.shape[1])


def _pad_rows8(k):
    """Passages padded with zero rows to a multiple of 8 (the kernels' granularity); the label
    padding marks those columns as ignored, and autograd drops their gradient rows."""
    extra = (-k.shape[0]) % 8
    return k if extra == 0 else torch.cat([k, k.new_zeros(extra, k.shape[1])], dim=0)


def fused_label_loss(q, k, labels, temperature: float, scores=None):
    """Label-matrix contrastive loss on the streaming kernels. ``labels [Q, K]``: 1 positive,
    0 negative, negative values ignored. Without ``scores``: multi-positive NCE
    ``mean_q(LSE_valid(s_q) − mean_{p ∈ pos(q)} s_qp)``; with ``scores``: soft-label cross-entropy
    against ``scores / sum(scores)`` over the non-ignored columns. Queries without a positive (or
    with a zero score sum) are skipped, as in lset/losses/contrastive.py:22-53. No host sync."""
    Q, K = labels.shape
    dev = q.device
    Kp = (K + 31) // 32 * 32
    lab8 = torch.full((Q, Kp), -1, dtype=torch.int8, device=dev)
    lab8[:, :K].copy_(labels)           # converts in the copy: no fp32 [Q, K] temporary
    labels = lab8[:, :K]
    any_valid = labels.max(dim=1).values >= 0      # row statistics without [Q, K] temporaries
    tw = None
    if scores is not None:
        tw = torch.zeros(Q, Kp, dtype=torch.float32, device=dev)
        tw[:, :K] = scores.to(dev, torch.float32)
        torch.nan_to_num_(tw, nan=0.0, posinf=0.0, neginf=0.0)   # "no teacher score": target 0
        tw[:, :K].masked_fill_(labels < 0, 0.0)
        tsum = tw.sum(dim=1)
        keep = (tsum > 0) & any_valid
        row_scale = 1.0 / tsum.clamp(min=1e-12)
    else:
        n_pos = labels.clamp(min=0).sum(dim=1, dtype=torch.int32)   # labels are -1 / 0 / 1 here
        keep = (n_pos > 0) & any_valid
        row_scale = 1.0 / n_pos.clamp(min=1).float()
    keepf = keep.float()
    row_w = keepf / keepf.sum().clamp(min=1.0)
    return _FusedLabelLoss.apply(q.contiguous(), _pad_rows8(k).contiguous(), lab8, tw,
                                 row_scale.contiguous(), row_w.contiguous(),
                                 1.0 / float(temperature))


# ------------------------------------------------------------------------------------------------
# Multi-positive NCE (every positive against the query's negatives only), and the int8-label
# "soft" / "cross" cross-entropies: the three loss types of lset/kernels/loss.py:1051-1089.
# ------------------------------------------------------------------------------------------------
def reference_switches_to_fused(num_queries: int, num_docs: int, loss_type: str = "multi") -> bool:
    """Sizes from which the reference replaces its eager label-matrix loss by its fused kernel, and
    with it the loss definition (lset/kernels/loss.py:37-55). Used only to keep the *semantics*
    aligned with the reference at every batch size; speed is not the criterion here."""
    if loss_type == "multi":
        return num_queries >= 2048 or (num_queries >= 1024 and num_docs >= 4096)
    return num_queries >= 2048 and num_docs >= 4096


def _pad_labels_int8(labels):
    Q, K = labels.shape
    Kp = (K + 31) // 32 * 32
    lab8 = torch.full((Q, Kp), -1, dtype=torch.int8, device=labels.device)
    lab8[:, :K].copy_(labels)
    return lab8


class _FusedMpNce(torch.autograd.Function):
    """loss = mean_{valid q} mean_{p ∈ pos(q)} softplus(LSE_{n ∈ neg(q)} s_qn − s_qp)."""

    @staticmethod
    def forward(ctx, q, k, labels8, pos_qi, pos_di, inv_t):
        M, D = q.shape
        N = k.shape[0]
        dev = q.device
        lib = nv.load()
        lib.lb_infonce_scratch_floats.restype = nv.c_ll
        scr = torch.empty(int(lib.lb_infonce_scratch_floats(nv.c_int(M), nv.c_int(N))),
                          dtype=torch.float32, device=dev)
        neg_lse = torch.empty(M, dtype=torch.float32, device=dev)
        unused = torch.zeros(1, dtype=torch.float32, device=dev)
        ones = torch.ones(M, dtype=torch.float32, device=dev)
        zeros = torch.zeros(M, dtype=torch.float32, device=dev)
        rc = lib.lb_label_loss_fwd(
            nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), nv.c_void_p(k.data_ptr()),
            nv.c_ll(k.stride(0)), nv.c_int(M), nv.c_int(N), nv.c_int(D), nv.c_float(inv_t),
            nv.c_void_p(labels8.data_ptr()), nv.c_ll(labels8.stride(0)), nv.c_void_p(None),
            nv.c_ll(0), nv.c_void_p(ones.data_ptr()), nv.c_void_p(zeros.data_ptr()), nv.c_int(1),
            nv.c_void_p(scr.data_ptr()), nv.c_void_p(neg_lse.data_ptr()),
            nv.c_void_p(unused.data_ptr()), nv.c_void_p(nv.status_word(dev).data_ptr()),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_label_loss_fwd")
        nv.count_launch(2)
        lab = labels8[:, :N]
        num_pos = (lab > 0).sum(dim=1)
        has_neg = (lab == 0).any(dim=1)
        valid = ((num_pos > 0) & has_neg).float()
        denom = valid.sum().clamp(min=1.0)
        num_pos_f = num_pos.clamp(min=1).float()
        # scores of the positive pairs: P row dot products (P is a few per query)
        pos_scores = (q[pos_qi].float() * k[pos_di].float()).sum(dim=1) * inv_t
        gap = neg_lse[pos_qi] - pos_scores
        per_pos = torch.nn.functional.softplus(gap)
        q_sum = torch.zeros(M, dtype=torch.float32, device=dev).index_add_(0, pos_qi, per_pos)
        loss = ((q_sum / num_pos_f) * valid).sum() / denom
        aux = torch.zeros(M, dtype=torch.float32, device=dev).index_add_(0, pos_qi,
                                                                          torch.sigmoid(gap))
        row_w = valid / (denom * num_pos_f)
        ctx.save_for_backward(q, k, labels8, neg_lse, aux, row_w)
        ctx.inv_t = inv_t
        return loss

    @staticmethod
    def backward(ctx, g):
        q, k, labels8, neg_lse, aux, row_w = ctx.saved_tensors
        inv_t = ctx.inv_t
        M, D = q.shape
        N = k.shape[0]
        coef = (g.float() * inv_t).reshape(1).contiguous()
        lib = nv.load()
        status = nv.status_word(q.device).data_ptr()

        def pgrad(c0, c1, W):
            rc = lib.lb_label_loss_pgrad(
                nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)),
                nv.c_void_p(k.data_ptr() + c0 * k.stride(0) * k.element_size()),
                nv.c_ll(k.stride(0)), nv.c_int(M), nv.c_int(c1 - c0), nv.c_int(D), nv.c_float(inv_t),
                nv.c_void_p(labels8.data_ptr() + c0), nv.c_ll(labels8.stride(0)), nv.c_void_p(None),
                nv.c_ll(0), nv.c_void_p(aux.data_ptr()), nv.c_void_p(row_w.data_ptr()), nv.c_int(1),
                nv.c_void_p(neg_lse.data_ptr()), nv.c_void_p(coef.data_ptr()),
                nv.c_void_p(W.data_ptr()), nv.c_ll(W.stride(0)), nv.c_void_p(status),
                nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_label_loss_pgrad")
            nv.count_launch()

        dq, dk = streamed_loss_backward(pgrad, q, k, ctx.needs_input_grad[0],
                                        ctx.needs_input_grad[1])
        return dq, dk, None, None, None, None


def fused_dense_loss(q, k, labels, scale: float, loss_type: str = "multi", pos_qi=None,
                     pos_di=None, pos_counts=None):
    """The reference's fused dense embedding loss (lset/kernels/loss.py:1051-1089) on the streaming
    tcgen05 kernels. ``labels [Q, K]`` int8-valued: > 0 positive (the value is the soft label for
    "soft" / "cross"), 0 negative, < 0 ignored. ``scale`` = 1 / temperature (Python float).

    * ``"multi"``: multi-positive NCE, ``mean_q mean_{p} softplus(LSE_neg(q) − s_qp)`` over queries
      that have a positive and a negative.
    * ``"soft"``:  ``mean_q (LSE_valid(q) − Σ_k (l_qk / Σ l_q) s_qk)`` over queries with Σ l_q > 0.
    * ``"cross"``: ``mean_q (Σ l_q · LSE_valid(q) − Σ_k l_qk s_qk)``.
    ``pos_qi`` / ``pos_di`` (indices of the positive pairs, as the collator provides them) avoid a
    ``nonzero`` on the label matrix; ``pos_counts`` is accepted for signature parity."""
    del pos_counts
    if loss_type not in ("multi", "soft", "cross"):
        raise ValueError(f"unknown loss_type {loss_type!r}")
    lab8 = _pad_labels_int8(labels.to(q.device))
    K = labels.shape[1]
    q, k = q.contiguous(), _pad_rows8(k).contiguous()
    if loss_type == "multi":
        if pos_qi is None or pos_di is None:
            pos_qi, pos_di = (lab8[:, :K] > 0).nonzero(as_tuple=True)
        return _FusedMpNce.apply(q, k, lab8, pos_qi.to(q.device).long(), pos_di.to(q.device).long(),
                                 float(scale))
    lab = lab8[:, :K]
    label_sum = lab.clamp(min=0).sum(dim=1).float()
    keep = (label_sum > 0).float()
    row_scale = 1.0 / label_sum.clamp(min=1e-9)
    row_w = keep / keep.sum().clamp(min=1.0)
    if loss_type == "cross":
        row_w = row_w * label_sum     # Σl·LSE − Σ l·s  =  Σl · (LSE − Σ (l/Σl)·s)
    return _FusedLabelLoss.apply(q, k, lab8, None, row_scale.contiguous(), row_w.contiguous(),
                                 float(scale))
