"""Cross-rank gathers of embeddings for global in-batch negatives.

``gather_with_grad`` keeps the reference's semantics (lset/distributed/gather.py:7-35): all-gather,
own shard passes gradient through, backward keeps only the local slice. It is meant for losses
that every rank evaluates on the full global score matrix.

``gather_for_local_rows`` is what this framework's task uses: every rank scores only its *own*
query rows against all gathered passages (1/W of the reference's redundant work); the backward
then sums each passage's gradient contributions from all ranks back to its owner with a
reduce-scatter. Both take an optional process group (the data-parallel group on a 2-D mesh).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group=None):
    if not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


class _GatherKeepLocal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        W, r = _world(group)
        ctx.rank, ctx.rows = r, x.shape[0]
        out = torch.empty(W * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        s = ctx.rank * ctx.rows
        return g[s:s + ctx.rows].contiguous(), None


class _GatherReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        W, r = _world(group)
        ctx.group, ctx.rank, ctx.rows, ctx.W = group, r, x.shape[0], W
        out = torch.empty(W * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if g.is_cuda:
            out = torch.empty(ctx.rows, *g.shape[1:], dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.SUM, group=ctx.group)
            return out, None
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)  # gloo has no reduce-scatter
        s = ctx.rank * ctx.rows
        return g[s:s + ctx.rows].contiguous(), None


def gather_with_grad(tensor, group=None):
    """All-gather along dim 0; gradient flows back to the local shard only."""
    if _world(group)[0] == 1:
        return tensor
    return _GatherKeepLocal.apply(tensor, group)


def gather_for_local_rows(tensor, group=None):
    """All-gather along dim 0 whose backward reduce-scatters (sums) gradients to the owners."""
    if _world(group)[0] == 1:
        return tensor
    return _GatherReduceScatter.apply(tensor, group)
