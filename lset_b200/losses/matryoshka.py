"""Matryoshka representation learning: the mean of the base loss over re-normalised prefix slices
of the embeddings (lset/losses/matryoshka.py:10-26). With ``labels`` the base loss is the
label-matrix contrastive loss, otherwise diagonal InfoNCE."""
from __future__ import annotations

from ..ops.pooling import normalize
from .contrastive import contrastive_loss
from .infonce import infonce_loss


def matryoshka_loss(query_embeds, doc_embeds, dims, temperature=0.02, labels=None, **kwargs):
    total = 0.0
    for d in dims:
        q = normalize(query_embeds[:, :d].contiguous())
        k = normalize(doc_embeds[:, :d].contiguous())
        if labels is not None:
            total = total + contrastive_loss(q, k, labels, temperature, **kwargs)
        else:
            total = total + infonce_loss(q, k, temperature, **kwargs)
    return total / len(dims)
