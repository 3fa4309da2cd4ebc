"""Sequence-parallel tensor parallelism with the collectives fused into the GEMMs.

Between the blocks the residual stream is sharded by *tokens* over the tensor-parallel ranks; a
column-parallel layer needs every token (all-gather → GEMM), a row-parallel layer produces partial
sums for every token (GEMM → reduce-scatter). On NVLink-connected GPUs both pairs run as ONE kernel:

* ``ag_linear``  — every rank publishes its token shard in a symmetric buffer; two extra warps of
  the GEMM CTAs pull the peers' rows over NVLink into a local ``[T, K]`` matrix while the tcgen05
  tiles consume them in pull order (``lb_gemm_bf16_ag``).
* ``linear_rs``  — the GEMM epilogue adds every fp32 output row straight into its owner's
  accumulator with ``red.global.add`` over NVLink (``lb_gemm_bf16_scatter``).

Their backward passes are each other's mirror image (the gradient of an all-gather is a
reduce-scatter and vice versa), so the same two kernels serve forward and backward. Ranks are
ordered by one device barrier per op (``symm.DeviceBarrier``: flags in symmetric memory, bounded
wait), enqueued on the compute stream; the GEMM kernels themselves never wait on another GPU.
Buffers are double-buffered by an epoch counter, which removes the need for a second "done
reading" barrier (see ``SPState``).

Without symmetric memory (CPU / gloo, or a GPU pair without peer access) the same functions fall
back to an explicit all-gather / reduce-scatter around a local GEMM, so the model plumbing is
testable on CPU. Counterpart of the reference's ``SequenceParallel`` + ``Colwise/RowwiseParallel``
styles (lset/distributed/tp.py:9-11, lset/models/decoder/qwen3/parallel_plan.py:34-50).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _native as nv
from ..ops._grads import main_grad_of
from ..ops.gemm import matmul_abt, wgrad_splits
from . import symm


def _capacity(rows: int) -> int:
    """Row capacity for ``rows``: headroom of a quarter, rounded up to 1024, so that batches of
    varying token counts reuse one allocation (symmetric allocations need a rendezvous)."""
    return ((rows + rows // 4 + 1023) // 1024) * 1024


class _AGBuf:
    """Double-buffered publication area for token shards of width K (any row count up to cap)."""

    def __init__(self, cap, K, world, device, group):
        self.cap = cap
        self.x_sym = [symm.SymmBuffer(cap * K, torch.bfloat16, device, group) for _ in range(2)]
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.device, self.world = device, world
        self._flags = {}   # rows -> (flags, epoch): the flag counts depend on the tile split

    def flags(self, rows):
        """Flag words and call count for this row count. A flag accumulates the items pulled over
        all calls that used it, so every row count keeps its own words and its own epoch."""
        ent = self._flags.get(rows)
        if ent is None:
            tiles = self.world * ((rows + 127) // 128)
            ent = self._flags[rows] = [torch.zeros(tiles, dtype=torch.int32, device=self.device), 0]
        return ent


class _RSBuf:
    """Double-buffered reduce-scatter areas of width N (any row count up to cap).

    bf16: every rank holds one slot per source rank; a GEMM *stores* its partial rows for rank r
    into its own slot of rank r's area and the owner sums the slots (no reductions on the wire,
    nothing to clear, fixed summation order). fp32: one accumulator that peers add into."""

    def __init__(self, cap, N, device, group, dtype=torch.float32):
        self.cap = cap
        self.dtype = dtype
        self.slots = dist.get_world_size(group) if dtype == torch.bfloat16 else 1
        self.rank = dist.get_rank(group)
        self.acc = [symm.SymmBuffer(cap * N * self.slots, dtype, device, group) for _ in range(2)]
        for a in self.acc:
            a.local.zero_()
        self.epoch = 0
        self._slot_ptrs = {}

    def slot_ptrs(self, half: int, rows: int, N: int):
        """Per destination rank, the address of this rank's slot in that rank's area (slots are
        ``rows * N`` elements apart: every rank of the group calls with the same ``rows``)."""
        key = (half, rows, N)
        arr = self._slot_ptrs.get(key)
        if arr is None:
            arr = self._slot_ptrs[key] = self.acc[half].offset_ptrs(self.rank * rows * N * 2)
        return arr


class SPState:
    """Per tensor-parallel group: rank bookkeeping and the symmetric buffers of the fused ops.

    Double buffering. Use ``e`` of a buffer pair touches half ``e & 1`` and contains exactly one
    ordering collective ``B_e``. All-gather: a rank rewrites half ``e & 1`` at use ``e + 2``, after
    it passed ``B_{e+1}``, which every peer joins only after its GEMM of use ``e`` (the reader of
    that half) is complete in stream order. Reduce-scatter: a rank clears its half right after
    reading it (after ``B_e``) and before it joins ``B_{e+1}``; peers add into that half again only
    at use ``e + 2``, i.e. after ``B_{e+1}``.
    """

    def __init__(self, group, device=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = None
        self.fused = False
        self._token = None
        # Reduce-scatter accumulators in bf16 (packed bf16x2 reductions over NVLink, half the bytes
        # of fp32; the same precision as a bf16 reduce-scatter of a collective library) or fp32.
        self.rs_bf16 = os.environ.get("LSET_B200_TP_RS_FP32", "0") != "1"
        if device is not None:
            self.bind(device)
        self._ag, self._rs, self._ag_epoch, self._retired = {}, {}, {}, []
        self._last_gather = None  # (x_shard, x_all) of the latest all-gather (q/k/v share it)

    def bind(self, device) -> None:
        """Fix the device (models are often sharded before they are moved to the GPU)."""
        device = torch.device(device)
        if self.device == device:
            return
        self.device = device
        self.fused = (device.type == "cuda" and 1 < self.world <= 8
                      and symm.enabled(self.world, device))
        self._token = None

    def token(self):
        """The group's device barrier (created on first use: a rendezvous of the group)."""
        if self._token is None:
            self._token = symm.DeviceBarrier(self.device, self.group)
        return self._token

    def barrier(self):
        self.token().sync()

    def ag_buf(self, rows, K) -> _AGBuf:
        b = self._ag.get(K)
        if b is None or b.cap < rows:
            # a larger batch than ever seen: new buffers (every rank takes this branch together,
            # the token count is the same on all ranks of the group). The old ones are kept: a
            # slower peer may still be reading them, and memory a peer maps must not be freed
            # under it.
            if b is not None:
                self._retired.append(b)
            b = self._ag[K] = _AGBuf(_capacity(rows), K, self.world, self.device, self.group)
            self._ag_epoch[K] = 0
        return b

    def rs_buf(self, rows, N) -> _RSBuf:
        dtype = torch.bfloat16 if self.rs_bf16 else torch.float32
        b = self._rs.get(N)
        if b is None or b.cap < rows or b.dtype != dtype:
            if b is not None:
                self._retired.append(b)
            b = self._rs[N] = _RSBuf(_capacity(rows), N, self.device, self.group, dtype)
            self.barrier()  # every rank's accumulators are cleared before anyone adds into them
        return b

    # ------------------------------------------------------------------ plain collectives
    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        out = x.new_empty(self.world * x.shape[0], *x.shape[1:])
        if x.is_cuda:
            dist.all_gather_into_tensor(out, x, group=self.group)
        else:
            dist.all_gather(list(out.chunk(self.world, dim=0)), x, group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        x = x.contiguous()
        rows = x.shape[0] // self.world
        if x.is_cuda:
            out = x.new_empty(rows, *x.shape[1:])
            dist.reduce_scatter_tensor(out, x, group=self.group)
            return out
        dist.all_reduce(x, group=self.group)  # gloo has no reduce-scatter
        return x[self.rank * rows:(self.rank + 1) * rows].clone()


# ---------------------------------------------------------------------- fused kernels
def _ag_gemm(st: SPState, x_shard, w, bias, b_mn: bool):
    """``(x_all, all_gather(x_shard) @ op(w))`` with the gather fused into the GEMM.
    ``op(w) = wᵀ`` for ``w [N, K]`` (``b_mn`` False) or ``w`` for ``w [K, N]`` (``b_mn`` True)."""
    rows, K = x_shard.shape
    W, rank = st.world, st.rank
    N = w.shape[1] if b_mn else w.shape[0]
    buf = st.ag_buf(rows, K)
    st._ag_epoch[K] += 1                       # which half of the publication area this use takes
    xs = buf.x_sym[st._ag_epoch[K] & 1]
    fl = buf.flags(rows)
    fl[1] += 1                                 # call count of these flag words
    xs.local[:rows * K].view(rows, K).copy_(x_shard)
    x_all = torch.empty(W * rows, K, dtype=torch.bfloat16, device=x_shard.device)
    x_all[rank * rows:(rank + 1) * rows].copy_(x_shard)  # own rows need no pull
    st.barrier()                                          # every shard is published
    y = torch.empty(W * rows, N, dtype=torch.bfloat16, device=x_shard.device)
    lib = nv.load()
    rc = lib.lb_gemm_bf16_ag(
        xs.c_ptr_array(), nv.c_void_p(x_all.data_ptr()), nv.c_void_p(w.data_ptr()),
        nv.c_void_p(y.data_ptr()), nv.c_int(rows), nv.c_int(W), nv.c_int(rank), nv.c_int(N),
        nv.c_int(K), nv.c_ll(K), nv.c_ll(w.stride(0)), nv.c_ll(N), nv.c_int(1 if b_mn else 0),
        nv.c_void_p(bias.data_ptr() if bias is not None else None),
        nv.c_void_p(fl[0].data_ptr()), nv.c_void_p(buf.counter.data_ptr()),
        ctypes.c_uint(fl[1]), nv.c_void_p(nv.status_word(x_shard.device).data_ptr()),
        nv.c_void_p(nv.stream_ptr()))
    nv.check_rc(rc, "lb_gemm_bf16_ag")
    nv.count_launch(1)
    return x_all, y


def _gemm_rs(st: SPState, a, w, b_mn: bool):
    """``reduce_scatter_rows(a @ op(w))`` with the reduction fused into the GEMM epilogue."""
    T, K = a.shape
    W = st.world
    rows = T // W
    N = w.shape[1] if b_mn else w.shape[0]
    buf = st.rs_buf(rows, N)
    buf.epoch += 1
    acc = buf.acc[buf.epoch & 1]
    lib = nv.load()
    if buf.dtype == torch.bfloat16:
        rc = lib.lb_gemm_bf16_push16(
            nv.c_void_p(a.data_ptr()), nv.c_void_p(w.data_ptr()),
            buf.slot_ptrs(buf.epoch & 1, rows, N), nv.c_int(W),
            nv.c_int(rows), nv.c_int(T), nv.c_int(N), nv.c_int(K), nv.c_ll(a.stride(0)),
            nv.c_ll(w.stride(0)), nv.c_ll(N), nv.c_int(0), nv.c_int(1 if b_mn else 0), nv.c_int(0),
            nv.c_void_p(nv.status_word(a.device).data_ptr()), nv.c_void_p(nv.stream_ptr()))
    else:
        rc = lib.lb_gemm_bf16_scatter(
            nv.c_void_p(a.data_ptr()), nv.c_void_p(w.data_ptr()), acc.c_ptr_array(), nv.c_int(W),
            nv.c_int(rows), nv.c_int(T), nv.c_int(N), nv.c_int(K), nv.c_ll(a.stride(0)),
            nv.c_ll(w.stride(0)), nv.c_ll(N), nv.c_int(0), nv.c_int(1 if b_mn else 0), nv.c_int(1),
            nv.c_int(0), nv.c_void_p(nv.status_word(a.device).data_ptr()),
            nv.c_void_p(nv.stream_ptr()))
    nv.check_rc(rc, "lb_gemm_bf16_scatter")
    nv.count_launch(1)
    st.barrier()                                          # every contribution has landed
    # read the reduced rows (fp32 accumulator: and leave it zero for its next use, in one pass)
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=a.device)
    n = rows * N
    if buf.dtype == torch.bfloat16:
        # sum of the W slots (each written by one rank's GEMM) in fp32, in slot order
        rc = lib.lb_take_sum(nv.c_void_p(acc.local.data_ptr()), nv.c_void_p(out.data_ptr()),
                             nv.c_ll(n), nv.c_int(W), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_take_sum")
        nv.count_launch(1)
    elif n % 8 == 0:
        rc = lib.lb_take_clear(nv.c_void_p(acc.local.data_ptr()), nv.c_void_p(out.data_ptr()),
                               nv.c_ll(n), nv.c_int(int(buf.dtype == torch.float32)),
                               nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_take_clear")
        nv.count_launch(1)
    else:
        used = acc.local[:n]
        out.copy_(used.view(rows, N))
        used.zero_()
    return out


def _fusable(st: SPState, *tensors) -> bool:
    return st.fused and all(t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()
                            and t.shape[-1] % 8 == 0 for t in tensors)


def _weight_grad(ctx_needs, w, dy, x):
    """dW = dyᵀ · x, added into ``w.main_grad`` when the sharding runtime provides one."""
    if not ctx_needs:
        return None
    main = main_grad_of(w)
    if dy.is_cuda and dy.dtype == torch.bfloat16:
        splits = wgrad_splits(w.shape[0], w.shape[1], x.shape[0])
        if main is not None:
            matmul_abt(dy, x, a_mn=True, b_mn=True, out=main, accumulate=True, splits=splits)
            return None
        return matmul_abt(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32,
                          splits=splits).to(w.dtype)
    return (dy.float().t() @ x.float()).to(w.dtype)


class _AGLinear(torch.autograd.Function):
    """``y[T, N_local] = all_gather(x_shard)[T, K] · wᵀ (+ bias)``; backward reduce-scatters dX."""

    @staticmethod
    def forward(ctx, x_shard, w, bias, st: SPState):
        st.bind(x_shard.device)
        cached = st._last_gather
        if cached is not None and cached[0] is x_shard:
            x_all = cached[1]   # a sibling projection of the same input already gathered it
            y = (matmul_abt(x_all, w, bias=bias) if x_all.is_cuda and x_all.dtype == torch.bfloat16
                 else torch.nn.functional.linear(x_all, w, bias))
        elif _fusable(st, x_shard, w):
            x_all, y = _ag_gemm(st, x_shard, w, bias, b_mn=False)
        else:
            x_all = st.all_gather_rows(x_shard)
            y = (matmul_abt(x_all, w, bias=bias) if x_all.is_cuda and x_all.dtype == torch.bfloat16
                 else torch.nn.functional.linear(x_all, w, bias))
        st._last_gather = (x_shard, x_all)
        ctx.save_for_backward(x_all, w)
        ctx.st, ctx.has_bias = st, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_all, w = ctx.saved_tensors
        st = ctx.st
        dy = dy.contiguous()
        if dy.is_cuda and dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        dx = None
        if ctx.needs_input_grad[0]:
            if _fusable(st, dy, w):
                dx = _gemm_rs(st, dy, w, b_mn=True)
            elif dy.is_cuda and dy.dtype == torch.bfloat16:
                dx = st.reduce_scatter_rows(matmul_abt(dy, w, b_mn=True))
            else:
                dx = st.reduce_scatter_rows(dy @ w)
        dw = _weight_grad(ctx.needs_input_grad[1], w, dy, x_all)
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None


class _LinearRS(torch.autograd.Function):
    """``y_shard[T/W, N] = reduce_scatter(x[T, K_local] · wᵀ)``; backward all-gathers dY."""

    @staticmethod
    def forward(ctx, x, w, st: SPState):
        st.bind(x.device)
        x = x.contiguous()
        if _fusable(st, x, w) and x.shape[0] % st.world == 0:
            y = _gemm_rs(st, x, w, b_mn=False)
        elif x.is_cuda and x.dtype == torch.bfloat16:
            y = st.reduce_scatter_rows(matmul_abt(x, w))
        else:
            y = st.reduce_scatter_rows(torch.nn.functional.linear(x, w))
        ctx.save_for_backward(x, w)
        ctx.st = st
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        st = ctx.st
        dy_shard = dy_shard.contiguous()
        if dy_shard.is_cuda and dy_shard.dtype != torch.bfloat16:
            dy_shard = dy_shard.to(torch.bfloat16)
        dx = None
        if _fusable(st, dy_shard, w) and ctx.needs_input_grad[0]:
            dy, dx = _ag_gemm(st, dy_shard, w, None, b_mn=True)
        else:
            dy = st.all_gather_rows(dy_shard)
            if ctx.needs_input_grad[0]:
                dx = (matmul_abt(dy, w, b_mn=True) if dy.is_cuda and dy.dtype == torch.bfloat16
                      else dy @ w)
        dw = _weight_grad(ctx.needs_input_grad[1], w, dy, x)
        return dx, dw, None


def ag_linear(x_shard, w, bias, st: SPState):
    return _AGLinear.apply(x_shard, w, bias, st)


def linear_rs(x, w, bias, st: SPState):
    y = _LinearRS.apply(x, w, st)
    return y if bias is None else y + bias  # added once, after the reduction


# ---------------------------------------------------------------------- residual-stream layout
class _ShardTokens(torch.autograd.Function):
    """Rows of this rank (after zero-padding to a multiple of the group size). Backward gathers the
    shards' gradients, so that what precedes (the embedding) sees the full gradient on every rank."""

    @staticmethod
    def forward(ctx, x, st: SPState):
        st.bind(x.device)
        T = x.shape[0]
        rows = (T + st.world - 1) // st.world
        ctx.st, ctx.T = st, T
        lo = st.rank * rows
        out = x.new_zeros(rows, *x.shape[1:])
        n = max(0, min(rows, T - lo))
        if n:
            out[:n].copy_(x[lo:lo + n])
        return out

    @staticmethod
    def backward(ctx, g):
        return ctx.st.all_gather_rows(g)[:ctx.T], None


class _UnshardTokens(torch.autograd.Function):
    """All-gather of the token shards. What follows is computed identically on every rank, so the
    gradient of a shard is simply this rank's slice."""

    @staticmethod
    def forward(ctx, x, T, st: SPState):
        ctx.st, ctx.rows = st, x.shape[0]
        return st.all_gather_rows(x)[:T]

    @staticmethod
    def backward(ctx, g):
        rows, st = ctx.rows, ctx.st
        lo = st.rank * rows
        out = g.new_zeros(rows, *g.shape[1:])
        n = max(0, min(rows, g.shape[0] - lo))
        if n:
            out[:n].copy_(g[lo:lo + n])
        return out, None, None


def shard_tokens(x, st: SPState):
    return _ShardTokens.apply(x, st)


def unshard_tokens(x, T: int, st: SPState):
    return _UnshardTokens.apply(x, T, st)


def pad_rows(x, total: int):
    """``x`` extended with zero rows to ``total`` rows (no copy when already that long)."""
    if x.shape[0] == total:
        return x
    return torch.cat([x, x.new_zeros(total - x.shape[0], *x.shape[1:])], dim=0)
