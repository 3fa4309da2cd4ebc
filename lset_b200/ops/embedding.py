"""Embedding lookup on the native gather kernel (sum of up to three tables, optional scale) with a
scatter-add backward into fp32 table gradients. Replaces aten embedding
(lset/models/decoder/qwen3/model.py:63, lset/models/encoder/bert/model.py:14-44)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native as nv
from ._grads import main_grad_of


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scale, ids0, tab0, ids1, tab1, ids2, tab2):
        T = ids0.numel()
        H = tab0.shape[1]
        out = torch.empty(T, H, dtype=tab0.dtype, device=tab0.device)
        rc = nv.load().lb_embedding_fwd(
            nv.c_void_p(ids0.data_ptr()), nv.c_void_p(tab0.data_ptr()),
            nv.c_void_p(nv.ptr(ids1)), nv.c_void_p(nv.ptr(tab1)),
            nv.c_void_p(nv.ptr(ids2)), nv.c_void_p(nv.ptr(tab2)),
            nv.c_void_p(out.data_ptr()), nv.c_ll(T), nv.c_int(H), nv.c_float(scale),
            nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_embedding_fwd")
        nv.count_launch()
        ctx.save_for_backward(ids0, ids1, ids2)
        ctx.tabs = (tab0, tab1, tab2)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dy):
        ids = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        T, H = dy.shape
        grads = []
        lib = nv.load()
        for k, tab in enumerate(ctx.tabs):
            if tab is None or not ctx.needs_input_grad[2 + 2 * k]:
                grads.append(None)
                continue
            main = main_grad_of(tab)
            dst = main if main is not None else torch.zeros(tab.shape, dtype=torch.float32,
                                                            device=tab.device)
            rc = lib.lb_embedding_bwd(nv.c_void_p(ids[k].data_ptr()), nv.c_void_p(dy.data_ptr()),
                                      nv.c_void_p(dst.data_ptr()), nv.c_ll(T), nv.c_int(H),
                                      nv.c_float(ctx.scale), nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_embedding_bwd")
            nv.count_launch()
            grads.append(None if main is not None else dst.to(tab.dtype))
        return None, None, grads[0], None, grads[1], None, grads[2]


class _EmbeddingEager(torch.autograd.Function):
    """CPU lookup whose backward adds the rows straight into the tables' fp32 accumulators
    (``index_add_``) when they have one, instead of materialising a dense zero-filled
    ``[vocab, H]`` gradient per call as aten's embedding backward does."""

    @staticmethod
    def forward(ctx, scale, n_tabs, *args):
        ids, tabs = args[:n_tabs], args[n_tabs:]
        out = tabs[0][ids[0]]
        for i, t in zip(ids[1:], tabs[1:]):
            out = out + t[i]
        ctx.save_for_backward(*ids)
        ctx.tabs, ctx.scale, ctx.n = tabs, scale, n_tabs
        return out * scale if scale != 1.0 else out

    @staticmethod
    def backward(ctx, dy):
        ids = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if ctx.scale != 1.0:
            dy2 = dy2 * ctx.scale
        grads = []
        for k, tab in enumerate(ctx.tabs):
            if not ctx.needs_input_grad[2 + ctx.n + k]:
                grads.append(None)
                continue
            main = main_grad_of(tab)
            dst = main if main is not None else torch.zeros_like(tab, dtype=torch.float32)
            dst.index_add_(0, ids[k].reshape(-1), dy2.to(dst.dtype))
            grads.append(None if main is not None else dst.to(tab.dtype))
        return (None, None) + (None,) * ctx.n + tuple(grads)


def embedding(ids, table, scale: float = 1.0, extra=()):
    """``scale * (table[ids] + sum(t[i] for i, t in extra))`` with the result shaped ``ids.shape + [H]``.

    ``extra`` holds up to two ``(ids, table)`` pairs (BERT position and token-type tables)."""
    native = nv.use_native(table) and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0
    if not native and not table.is_cuda and torch.is_grad_enabled() and any(
            t.requires_grad for t in (table, *[t for _, t in extra])):
        all_ids = [ids] + [i.expand_as(ids) for i, _ in extra]
        out = _EmbeddingEager.apply(float(scale), len(all_ids),
                                    *[i.to(torch.int64) for i in all_ids], table,
                                    *[t for _, t in extra])
        return out
    if not native or len(extra) > 2:
        out = F.embedding(ids, table)
        for i, t in extra:
            out = out + F.embedding(i, t)
        return out * scale if scale != 1.0 else out
    dev = table.device
    flat = [ids.reshape(-1).to(device=dev, dtype=torch.int64).contiguous()]
    tabs = [table]
    for i, t in extra:
        flat.append(i.expand_as(ids).reshape(-1).to(device=dev, dtype=torch.int64).contiguous())
        tabs.append(t)
    while len(flat) < 3:
        flat.append(None)
        tabs.append(None)
    out = _Embedding.apply(float(scale), flat[0], tabs[0], flat[1], tabs[1], flat[2], tabs[2])
    return out.view(*ids.shape, table.shape[1])
