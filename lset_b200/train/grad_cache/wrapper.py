"""GradCache: contrastive batches larger than activation memory allows.

Three passes (lset/train/grad_cache/wrapper.py:73-315): (1) embed every minibatch without
autograd, remembering the random state; (2) compute the loss on the cached embeddings as leaves
and take the gradient with respect to them; (3) re-encode every minibatch with autograd under the
remembered random state and back-propagate ``<embedding, cached gradient> * grad_output``.
The loss is the task's rank-local share (``BiEncoderTask.loss_from_embeddings``), so under data
parallelism pass 2 contains the cross-rank gather and its reduce-scatter backward.
"""
from __future__ import annotations

from typing import Optional

import torch

from .minibatch_backward import MinibatchBackward
from .planner import plan_minibatches, sequence_lengths, slice_feature
from .rand_context import RandContext


class GradCacheWrapper:
    def __init__(self, task, chunk_size: Optional[int] = 16, token_budget: Optional[int] = None,
                 selective_keep: float = 1.0, store=None):
        self.task = task
        self.chunk_size = chunk_size
        self.token_budget = token_budget
        self.selective_keep = selective_keep  # accepted for configuration parity; all samples replay
        self.store = store

    # -- pass 1 ------------------------------------------------------------------------------
    def _embed_no_grad(self, model, feature, plan, n_real):
        lens = sequence_lengths(feature) if "cu_seqlens" in feature else None
        leaves, states = [], []
        for i, (b, e) in enumerate(plan):
            sub = slice_feature(feature, b, e, lens)
            states.append(RandContext(sub["input_ids"]))
            with torch.no_grad():
                emb = self.task.encode(model, sub)
            if i < n_real:
                leaves.append(emb.detach().requires_grad_())
        return leaves, states

    # -- pass 3 ------------------------------------------------------------------------------
    def _replay(self, model, feature, plan, n_real, states, grads, runtime, grad_output, last_flags):
        lens = sequence_lengths(feature) if "cu_seqlens" in feature else None
        for i, (b, e) in enumerate(plan):
            sub = slice_feature(feature, b, e, lens)
            with states[i]:
                emb = self.task.encode(model, sub)
            g = grads[i] if i < n_real else torch.zeros_like(emb)
            surrogate = (emb.float() * g.float().to(emb.device)).sum() * grad_output
            runtime.backward(surrogate, last_flags[i])

    def __call__(self, model, query_batch, doc_batch, neg_batch=None, labels=None, scores=None,
                 is_ga_boundary: bool = True, grad_output: float = 1.0):
        runtime = MinibatchBackward.for_model(model, is_ga_boundary=is_ga_boundary, store=self.store)
        feats = [f for f in (query_batch, doc_batch, neg_batch) if f is not None]
        plans = [plan_minibatches(f, self.chunk_size, self.token_budget) for f in feats]
        plans, real = runtime.align_minibatches(plans)

        cached = [self._embed_no_grad(model, f, p, n) for f, p, n in zip(feats, plans, real)]
        full = [torch.cat(leaves, dim=0) for leaves, _ in cached]
        q_emb, d_emb = full[0], full[1]
        n_emb = full[2] if len(full) > 2 else None
        loss = self.task.loss_from_embeddings(q_emb, d_emb, n_emb, labels, scores)
        wrt = [leaf for leaves, _ in cached for leaf in leaves]
        scale_params = [p for p in self.task.parameters() if p.requires_grad]
        all_grads = torch.autograd.grad(loss, wrt + scale_params, allow_unused=True)
        for p, g in zip(scale_params, all_grads[len(wrt):]):
            if g is not None:
                g = g * grad_output
                if hasattr(p, "main_grad"):
                    p.main_grad.add_(g.to(p.main_grad.dtype))
                else:
                    p.grad = g if p.grad is None else p.grad + g
        leaf_grads = list(all_grads[:len(wrt)])

        total = sum(len(p) for p in plans)
        done = 0
        with runtime.context():
            k = 0
            for (leaves, states), f, p, n in zip(cached, feats, plans, real):
                grads = leaf_grads[k:k + len(leaves)]
                k += len(leaves)
                flags = [(done + i) == total - 1 for i in range(len(p))]
                self._replay(model, f, p, n, states, grads, runtime, grad_output, flags)
                done += len(p)
        runtime.finalize(list(model.parameters()))
        return loss.detach()
