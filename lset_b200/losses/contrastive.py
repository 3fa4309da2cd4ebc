"""Label-matrix contrastive loss: multi-positive NCE and soft-label cross-entropy
(semantics of lset/losses/contrastive.py:14-53). Labels: 1 = positive, 0 = negative, -1 = ignore.

* multi-positive: ``mean_q( -mean_{p in pos(q)} sim[q,p] + logsumexp_{valid} sim[q,:] )``
* soft labels (``scores`` given): targets are the row-normalised softmax of the teacher scores over
  valid entries; loss is the cross-entropy against the log-softmax over valid entries.
Queries without a positive (or without a valid column) are skipped; with none left the result is a
zero that still carries gradient."""
from __future__ import annotations

import torch

from ..ops.loss import similarity


def _zero_with_grad(*tensors):
    return sum((t.float() * 0.0).sum() for t in tensors)


def contrastive_loss(query_embeds, doc_embeds, labels, temperature=0.02, scores=None, scale=None):
    s = (1.0 / temperature) if scale is None else scale
    sim = similarity(query_embeds, doc_embeds) * s
    labels = labels.to(sim.device)
    valid = labels >= 0
    masked = sim.masked_fill(~valid, float("-inf"))
    if scores is not None:
        sc = scores.to(sim.device).float().masked_fill(~valid, float("-inf"))
        keep = valid.any(dim=1)
        if not keep.any():
            return _zero_with_grad(query_embeds, doc_embeds)
        target = torch.softmax(sc[keep], dim=1)
        logp = torch.log_softmax(masked[keep], dim=1)
        per_q = -(target * logp.masked_fill(~valid[keep], 0.0)).sum(dim=1)
        return per_q.mean()
    pos = labels > 0
    n_pos = pos.sum(dim=1)
    keep = n_pos > 0
    if not keep.any():
        return _zero_with_grad(query_embeds, doc_embeds)
    pos_term = (sim * pos).sum(dim=1) / n_pos.clamp(min=1)
    lse = torch.logsumexp(masked, dim=1)
    per_q = lse - pos_term
    return per_q[keep].mean()
