"""In-batch-negative InfoNCE with optional top-K hard-negative truncation
(semantics of lset/losses/infonce.py:9-32). ``doc_embeds`` may hold more rows than queries; the
extra rows are pure negatives. ``target_offset`` shifts the positive column (rank offset when the
documents are a cross-rank gather and the queries are local)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops.loss import fused_infonce, fused_infonce_supported, similarity


def infonce_loss(query_embeds, doc_embeds, temperature=0.02, top_k=None, target_offset: int = 0):
    if (top_k is None and isinstance(temperature, (int, float))
            and fused_infonce_supported(query_embeds, doc_embeds)):
        # streaming kernel: the score matrix is never written to memory in fp32
        return fused_infonce(query_embeds, doc_embeds, float(temperature), target_offset)
    scale = 1.0 / temperature
    sim = similarity(query_embeds, doc_embeds) * scale
    B = query_embeds.shape[0]
    target = torch.arange(B, device=sim.device) + target_offset
    if top_k is not None and top_k < sim.shape[1] - 1:
        pos = sim.gather(1, target[:, None])
        neg = sim.scatter(1, target[:, None], float("-inf"))
        hard = neg.topk(top_k, dim=1).values
        logits = torch.cat([pos, hard], dim=1)
        return F.cross_entropy(logits, torch.zeros(B, dtype=torch.long, device=sim.device))
    return F.cross_entropy(sim, target)
