"""Pipeline parallelism: split points and per-stage module names (the planning helpers of
lset/distributed/pp.py:4-33), plus a fill-drain runner that actually executes the stages
(``PipelineRunner``), which the reference does not have. The training engine keeps ``pp_size`` at
1, as the reference does; the runner is a library component driven directly (see its docstring).
"""
from __future__ import annotations

from typing import Dict, List

import torch.nn as nn


def get_pp_split_points(num_layers: int, pp_size: int) -> Dict[str, str]:
    """``{"layers.k": "BEGINNING"}`` for the first layer of every stage but the first."""
    if pp_size <= 1:
        return {}
    per = num_layers // pp_size
    extra = num_layers % pp_size
    points, start = {}, 0
    for stage in range(pp_size - 1):
        start += per + (1 if stage < extra else 0)
        points[f"layers.{start}"] = "BEGINNING"
    return points


def get_stage_module_names(num_layers: int, pp_size: int, has_embeddings_name: str = "embed_tokens",
                           final_norm_name: str = "norm") -> List[List[str]]:
    """Module names per stage: embeddings on the first stage, the final norm on the last."""
    per = num_layers // max(1, pp_size)
    extra = num_layers % max(1, pp_size)
    stages, start = [], 0
    for stage in range(max(1, pp_size)):
        n = per + (1 if stage < extra else 0)
        names = [f"layers.{i}" for i in range(start, start + n)]
        if stage == 0:
            names.insert(0, has_embeddings_name)
        if stage == pp_size - 1 or pp_size <= 1:
            names.append(final_norm_name)
        stages.append(names)
        start += n
    return stages


def stage_layer_range(num_layers: int, pp_size: int, stage: int):
    """``(lo, hi)``: the decoder layers of ``stage`` under the split of ``get_pp_split_points``."""
    per, extra = divmod(num_layers, max(1, pp_size))
    lo = stage * per + min(stage, extra)
    return lo, lo + per + (1 if stage < extra else 0)


class PipelineRunner:
    """Fill-drain (GPipe) schedule for a decoder embedder split over a pipeline group.

    Beyond what the reference ships (it stops at the split-point helpers, lset/distributed/pp.py:4-33):
    rank ``s`` of ``pp_group`` keeps the layers of stage ``s`` (plus the embeddings on the first and
    the final norm on the last stage) and drops the rest. ``encode`` runs every micro-batch forward —
    the open residual stream ``(branch, residual)`` travels between neighbouring stages with
    point-to-point sends — and returns the final hidden states on the last stage. ``backward`` takes
    the gradients of those hidden states (from a contrastive loss over *all* micro-batches, which
    is why the schedule drains before it turns around) and runs the stages in reverse.

    Every rank of the group must be given the same micro-batches (token ids and sequence
    boundaries): each stage needs positions and attention plans, and shapes are known without a
    handshake. Works on any backend with send/recv (gloo on the CPU, NCCL on GPUs).
    """

    def __init__(self, model, pp_group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = pp_group
        self.size = dist.get_world_size(pp_group)
        self.stage = dist.get_rank(pp_group)
        self.model = model
        n = len(model.layers)
        if self.size > n:
            raise ValueError(f"{self.size} pipeline stages for {n} layers")
        self.lo, self.hi = stage_layer_range(n, self.size, self.stage)
        self.first, self.last = self.stage == 0, self.stage == self.size - 1
        # drop what other stages own (parameters and their optimizer state live there)
        for i in range(n):
            if not self.lo <= i < self.hi:
                model.layers[i] = _Dropped()
        if not self.first:
            model.embed_tokens = _Dropped()
        if not self.last:
            model.norm = _Dropped()
        self._saved = []

    def _peer(self, stage: int) -> int:
        return self.dist.get_global_rank(self.group, stage) if self.group is not None else stage

    def _ctx(self, mb):
        from ..models.layers import make_stream_ctx

        return make_stream_ctx(mb["input_ids"], mb.get("attention_mask"), mb.get("position_ids"),
                               mb.get("cu_seqlens"), mb.get("max_seqlen"))

    def encode(self, microbatches):
        """Forward of every micro-batch. Returns the list of hidden states (last stage) or an empty
        list (other stages); keeps what ``backward`` needs."""
        import torch

        dist, m = self.dist, self.model
        p = next(m.parameters())
        H = m.config.hidden_size
        self._saved, outs = [], []
        for mb in microbatches:
            ids = mb["input_ids"].to(p.device)
            ctx = self._ctx({**mb, "input_ids": ids})
            T = ids.numel()
            stream_in = None
            if not self.first:
                stream_in = [torch.empty(T, H, dtype=p.dtype, device=p.device) for _ in range(2)]
                for t in stream_in:
                    dist.recv(t, src=self._peer(self.stage - 1), group=self.group)
                    t.requires_grad_()
            out = m.run_stage(ids.reshape(-1), stream_in, ctx, self.lo, self.hi)
            if self.last:
                if ctx.padded_shape is not None:
                    out = out.view(*ctx.padded_shape, H)
                outs.append(out)
                self._saved.append((stream_in, [out]))
            else:
                for t in out:
                    dist.send(t.detach().contiguous(), dst=self._peer(self.stage + 1),
                              group=self.group)
                self._saved.append((stream_in, list(out)))
        return outs

    def backward(self, hidden_grads=None):
        """Backward of every micro-batch in reverse order. ``hidden_grads``: on the last stage, one
        gradient per hidden-state tensor returned by ``encode``."""
        import torch

        dist = self.dist
        for i in reversed(range(len(self._saved))):
            stream_in, outs = self._saved[i]
            if self.last:
                grads = [hidden_grads[i].reshape(outs[0].shape)]
            else:
                grads = [torch.empty_like(t) for t in outs]
                for g in grads:
                    dist.recv(g, src=self._peer(self.stage + 1), group=self.group)
            torch.autograd.backward(outs, grads)
            if not self.first:
                for t in stream_in:
                    g = t.grad if t.grad is not None else torch.zeros_like(t)
                    dist.send(g.contiguous(), dst=self._peer(self.stage - 1), group=self.group)
        self._saved = []


class _Dropped(nn.Module):
    """Placeholder for a module that lives on another pipeline stage."""

    def forward(self, *a, **k):
        raise RuntimeError("this module belongs to another pipeline stage")
