"""Dispatcher between the streaming fused loss kernel and the dense label-matrix loss
(cf. lset/losses/fused_contrastive.py:16-59). The streaming kernel covers the diagonal-target
InfoNCE case; label matrices with several positives or teacher scores use the dense formulation on
top of the tcgen05 similarity product."""
from __future__ import annotations

from .contrastive import contrastive_loss


def fused_contrastive_loss(query_embeds, doc_embeds, labels, temperature=0.02, scores=None,
                           pos_qi=None, pos_di=None, pos_counts=None, scale=None):
    return contrastive_loss(query_embeds, doc_embeds, labels, temperature, scores, scale=scale)
