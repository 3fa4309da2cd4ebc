"""Post-pooling dense projection (EmbeddingGemma's ``2_Dense`` / ``3_Dense`` sentence-transformers
modules): bias-free linear maps applied to the pooled embedding before normalisation.

The reference ships the loader (lset/models/decoder/gemma/weights.py:30-36) and a registry slot
(``ModelSpec.post_pooling_fn``, lset/models/registry.py:15) without using either; here the slot
holds a factory ``model_dir -> module or None`` and the training task, the chunked encoder and the
MTEB wrapper apply the module between pooling and L2 normalisation.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn

from ..ops import gemm as gemm_ops


class PostPoolingDense(nn.Module):
    """``x -> x @ W0ᵀ -> ... @ Wnᵀ`` with frozen matrices (buffers, so they follow ``.to()``)."""

    def __init__(self, matrices: Sequence[torch.Tensor]):
        super().__init__()
        self.n = len(matrices)
        for i, w in enumerate(matrices):
            self.register_buffer(f"w{i}", w.detach().clone())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for i in range(self.n):
            w = getattr(self, f"w{i}")
            x = gemm_ops.linear(x, w.to(x.dtype) if w.dtype != x.dtype else w)
        return x

    @property
    def out_features(self) -> int:
        return int(getattr(self, f"w{self.n - 1}").shape[0])


def gemma_post_pooling(model_dir) -> Optional[PostPoolingDense]:
    """Module for the dense layers stored next to an EmbeddingGemma checkpoint, or None."""
    from .weights import load_gemma_projection

    if model_dir is None:
        return None
    mats = load_gemma_projection(model_dir)
    return PostPoolingDense(mats) if mats else None
