"""Label-matrix contrastive loss: multi-positive NCE and soft-label cross-entropy
(semantics of lset/losses/contrastive.py:14-53). Labels: 1 = positive, 0 = negative, -1 = ignore.

* multi-positive: ``mean_q( -mean_{p in pos(q)} sim[q,p] + logsumexp_{valid} sim[q,:] )``
* soft labels (``scores`` given): targets are the teacher scores over the non-ignored columns,
  normalised to sum to one; loss is ``logsumexp_{valid} sim[q,:] - sum_k target[q,k] sim[q,k]``.
  Non-finite scores mean "no teacher score": target 0. (The reference leaves the collator's -inf
  fill for other samples' documents in the targets, lset/train/data/collator.py:190-199 with
  lset/losses/contrastive.py:26-38, which makes every row's target sum -inf and the loss of a
  scored dataset identically zero.)
Queries without a positive (resp. with a zero score sum) or without a valid column are skipped;
with none left the result is a zero that still carries gradient. bf16 CUDA inputs with a Python
float temperature run on the streaming tensor-core kernels (``ops.loss.fused_label_loss``), which
never materialise the score matrix."""
from __future__ import annotations

import torch

from ..ops.loss import fused_label_loss, fused_label_loss_supported, similarity


def _zero_with_grad(*tensors):
    return sum((t.float() * 0.0).sum() for t in tensors)


def contrastive_loss(query_embeds, doc_embeds, labels, temperature=0.02, scores=None, scale=None):
    if (scale is None and isinstance(temperature, (int, float))
            and fused_label_loss_supported(query_embeds, doc_embeds)):
        return fused_label_loss(query_embeds, doc_embeds, labels, float(temperature), scores)
    s = (1.0 / temperature) if scale is None else scale
    sim = similarity(query_embeds, doc_embeds) * s
    labels = labels.to(sim.device)
    valid = labels >= 0
    masked = sim.masked_fill(~valid, float("-inf"))
    if scores is not None:
        # "no teacher score" entries (the collator fills documents of other samples with -inf)
        # are in-batch negatives with target 0
        target = torch.nan_to_num(scores.to(sim.device).float(), nan=0.0, posinf=0.0, neginf=0.0)
        target = target.masked_fill(~valid, 0.0)
        tsum = target.sum(dim=1)
        keep = (tsum > 0) & valid.any(dim=1)
        if not keep.any():
            return _zero_with_grad(query_embeds, doc_embeds)
        target = target / tsum.clamp(min=1e-12).unsqueeze(1)
        per_q = torch.logsumexp(masked, dim=1) - (target * sim).sum(dim=1)
        return per_q[keep].mean()
    pos = labels > 0
    n_pos = pos.sum(dim=1)
    keep = n_pos > 0
    if not keep.any():
        return _zero_with_grad(query_embeds, doc_embeds)
    pos_term = (sim * pos).sum(dim=1) / n_pos.clamp(min=1)
    lse = torch.logsumexp(masked, dim=1)
    per_q = lse - pos_term
    return per_q[keep].mean()
