"""Cross-rank InfoNCE on peer memory: local queries against every rank's passages.

Forward: each rank publishes its passage embeddings in a symmetric buffer; one kernel pulls the
peers' rows over NVLink (two extra warps per CTA) into a local ``[W * B, D]`` buffer while the
tcgen05 tiles of ``Q · Kᵀ`` consume them in pull order with an online logsumexp — the all-gather is
fused into the similarity GEMM, and no score matrix is written. Backward: the softmax gradient is
recomputed as a bf16 ``W`` one column panel at a time (a panel never spans two ranks' passages and
is capped at 64 MB), ``dQ`` accumulates ``W · K`` over the panels locally,
and each panel's ``dK = Wᵀ · Q`` is produced by a GEMM whose epilogue adds every row straight into
its *owner's* fp32 buffer with ``red.global.add`` over NVLink — the reduce-scatter is fused into
the GEMM.

Ranks are ordered with two device barriers per step (passages published and accumulators cleared;
all dK contributions landed): one-warp kernels with a bounded wait on flags in symmetric memory,
enqueued on the compute stream, so the GEMM kernels themselves never wait on another GPU. Same value and gradients as
``gather_for_local_rows`` + ``infonce_loss``; replaces the reference's ``all_gather`` + loss kernel
(lset/distributed/gather.py:7-35, lset/kernels/loss.py).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _native as nv
from ..ops.gemm import matmul_abt
from . import symm

_state = {}


class _Buffers:
    """Per (group, n_local, D) symmetric and local buffers, reused across steps."""

    def __init__(self, n_local: int, D: int, device, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        # two passage buffers used alternately: a rank may publish step t+1 while a slow peer is
        # still pulling step t, so no "done reading" barrier is needed
        self.k_sym = [symm.SymmBuffer(n_local * D, torch.bfloat16, device, group) for _ in range(2)]
        self.dk_sym = symm.SymmBuffer(n_local * D, torch.float32, device, group)
        self.k_all = torch.empty(self.world * n_local, D, dtype=torch.bfloat16, device=device)
        tiles = self.world * ((n_local + 255) // 256)
        self.flags = torch.zeros(tiles, dtype=torch.int32, device=device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.barrier = symm.DeviceBarrier(device, group)
        self.epoch = 0

    def order_ranks(self):
        self.barrier.sync()


def _buffers(n_local, D, device, group) -> _Buffers:
    key = (id(group), n_local, D, device.index)
    b = _state.get(key)
    if b is None:
        b = _Buffers(n_local, D, device, group)
        _state[key] = b
    return b


def supported(q, d, group=None) -> bool:
    if not (dist.is_available() and dist.is_initialized()):
        return False
    W = dist.get_world_size(group)
    return (symm.enabled(W, q.device) and 1 < W <= 8 and q.dtype == torch.bfloat16
            and d.dtype == torch.bfloat16 and q.shape[1] % 8 == 0 and d.shape[0] % 8 == 0
            and q.shape[1] == d.shape[1])


class _CrossRankInfoNCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, d, inv_t, group):
        B, D = q.shape
        n_local = d.shape[0]
        buf = _buffers(n_local, D, q.device, group)
        W, rank = buf.world, buf.rank
        lib = nv.load()
        lib.lb_infonce_xrank_scratch_floats.restype = nv.c_ll
        buf.epoch += 1
        ksym = buf.k_sym[buf.epoch & 1]
        ksym.local.view(n_local, D).copy_(d)
        buf.k_all[rank * n_local:(rank + 1) * n_local].copy_(d)   # own rows need no pull
        buf.dk_sym.local.zero_()               # owners' dK accumulators start at zero
        buf.order_ranks()                      # passages published and accumulators cleared everywhere
        scr = torch.empty(int(lib.lb_infonce_xrank_scratch_floats(
            nv.c_int(B), nv.c_int(n_local), nv.c_int(W))), dtype=torch.float32, device=q.device)
        lse = torch.empty(B, dtype=torch.float32, device=q.device)
        loss_sum = torch.zeros(1, dtype=torch.float32, device=q.device)
        rc = lib.lb_infonce_fwd_xrank(
            nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), ksym.c_ptr_array(),
            nv.c_void_p(buf.k_all.data_ptr()), nv.c_ll(D), nv.c_int(B), nv.c_int(n_local),
            nv.c_int(W), nv.c_int(rank), nv.c_int(D), nv.c_float(inv_t), nv.c_ll(rank * n_local),
            nv.c_void_p(scr.data_ptr()), nv.c_void_p(lse.data_ptr()),
            nv.c_void_p(loss_sum.data_ptr()), nv.c_void_p(buf.flags.data_ptr()),
            nv.c_void_p(buf.counter.data_ptr()), ctypes.c_uint(buf.epoch),
            nv.c_void_p(nv.status_word(q.device).data_ptr()), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_infonce_fwd_xrank")
        nv.count_launch(2)
        ctx.save_for_backward(q, lse)
        ctx.meta = (inv_t, group, n_local)
        return loss_sum[0] / float(W * B)

    @staticmethod
    def backward(ctx, g):
        q, lse = ctx.saved_tensors
        inv_t, group, n_local = ctx.meta
        B, D = q.shape
        buf = _buffers(n_local, D, q.device, group)
        W, rank = buf.world, buf.rank
        N = W * n_local
        lib = nv.load()
        coef = (g.float() * (inv_t / float(W * B))).reshape(1).contiguous()
        from ..ops.loss import PANEL_BYTES, panel_cols

        Bp = (B + 7) // 8 * 8
        status = nv.status_word(q.device).data_ptr()
        qp = q if Bp == B else torch.cat([q, q.new_zeros(Bp - B, D)])
        if Bp * N * 2 <= PANEL_BYTES:
            # the whole probability gradient fits one panel: one recompute over every rank's
            # passages, one dQ product, and one dK product whose epilogue scatters each block of
            # rows to its owner (three launches whatever the number of ranks)
            Wm = torch.empty(Bp, N, dtype=torch.bfloat16, device=q.device)
            if Bp != B:
                Wm[B:].zero_()
            rc = lib.lb_infonce_pgrad(
                nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)), nv.c_void_p(buf.k_all.data_ptr()),
                nv.c_ll(D), nv.c_int(B), nv.c_int(N), nv.c_int(D), nv.c_float(inv_t),
                nv.c_ll(rank * n_local), nv.c_void_p(lse.data_ptr()), nv.c_void_p(coef.data_ptr()),
                nv.c_void_p(Wm.data_ptr()), nv.c_ll(N), nv.c_void_p(status),
                nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_infonce_pgrad")
            dq = matmul_abt(Wm[:B], buf.k_all, b_mn=True)
            rc = lib.lb_gemm_bf16_scatter(
                nv.c_void_p(Wm.data_ptr()), nv.c_void_p(qp.data_ptr()), buf.dk_sym.c_ptr_array(),
                nv.c_int(W), nv.c_int(n_local), nv.c_int(N), nv.c_int(D), nv.c_int(Bp), nv.c_ll(N),
                nv.c_ll(D), nv.c_ll(D), nv.c_int(1), nv.c_int(1), nv.c_int(1), nv.c_int(0),
                nv.c_void_p(status), nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_gemm_bf16_scatter")
            nv.count_launch(3)
            buf.order_ranks()                  # every contribution has landed
            dk = buf.dk_sym.local.view(n_local, D).to(torch.bfloat16)
            return dq, dk, None, None
        step = min(n_local, panel_cols(B, N))
        Wm = torch.empty(Bp, step, dtype=torch.bfloat16, device=q.device)
        if Bp != B:
            Wm[B:].zero_()
        dq32 = None
        for pk in range(W):
            peer = (rank + pk) % W                    # own passages first, then the peers in turn
            for s0 in range(0, n_local, step):
                n = min(step, n_local - s0)
                c0 = peer * n_local + s0              # first global column of the panel
                Wp = Wm if n == step else Wm[:, :n]
                k_panel = buf.k_all[c0:c0 + n]
                rc = lib.lb_infonce_pgrad(
                    nv.c_void_p(q.data_ptr()), nv.c_ll(q.stride(0)),
                    nv.c_void_p(k_panel.data_ptr()), nv.c_ll(D), nv.c_int(B), nv.c_int(n),
                    nv.c_int(D), nv.c_float(inv_t), nv.c_ll(rank * n_local - c0),
                    nv.c_void_p(lse.data_ptr()), nv.c_void_p(coef.data_ptr()),
                    nv.c_void_p(Wp.data_ptr()), nv.c_ll(Wp.stride(0)), nv.c_void_p(status),
                    nv.c_void_p(nv.stream_ptr()))
                nv.check_rc(rc, "lb_infonce_pgrad")
                if dq32 is None:
                    dq32 = matmul_abt(Wp[:B], k_panel, b_mn=True, out_dtype=torch.float32)
                else:
                    matmul_abt(Wp[:B], k_panel, b_mn=True, out=dq32, accumulate=True)
                # dK of the panel: every rank adds its contribution into the owner's buffer
                # (cleared in forward), rows s0 .. s0 + n of that rank's passages
                owner = (ctypes.c_void_p * 1)(buf.dk_sym.peer_ptrs[peer] + 4 * s0 * D)
                rc = lib.lb_gemm_bf16_scatter(
                    nv.c_void_p(Wp.data_ptr()), nv.c_void_p(qp.data_ptr()), owner,
                    nv.c_int(1), nv.c_int(n), nv.c_int(n), nv.c_int(D), nv.c_int(Bp),
                    nv.c_ll(Wp.stride(0)), nv.c_ll(D), nv.c_ll(D), nv.c_int(1), nv.c_int(1),
                    nv.c_int(0), nv.c_int(0), nv.c_void_p(status), nv.c_void_p(nv.stream_ptr()))
                nv.check_rc(rc, "lb_gemm_bf16_scatter")
                nv.count_launch(3)
        dq = dq32.to(q.dtype)
        buf.order_ranks()                      # every contribution has landed
        dk = buf.dk_sym.local.view(n_local, D).to(torch.bfloat16)
        return dq, dk, None, None


def cross_rank_infonce(q, d, temperature: float, group=None):
    """This rank's share of the global InfoNCE loss (shares sum to the global mean)."""
    return _CrossRankInfoNCE.apply(q.contiguous(), d.contiguous(), 1.0 / float(temperature), group)
