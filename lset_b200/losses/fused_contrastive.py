"""Dispatcher between the streaming fused loss kernels and the dense label-matrix loss
(cf. lset/losses/fused_contrastive.py:16-59).

Both branches stream on the tcgen05 kernels for bf16 CUDA embeddings; what the dispatcher decides
is the loss *definition*. The reference's fused kernel implements ``loss_type`` "multi" as
multi-positive NCE against the negatives only (plus "soft" / "cross"), and the reference switches
to it only from a batch-size threshold, with the positive-pair indices given and no teacher scores
(lset/kernels/loss.py:37-55, lset/losses/fused_contrastive.py:30-35). The same rule is applied here
(``num_queries`` = the global number of queries when the caller scores a shard of the rows), so a
run produces the reference's loss values at every size. ``force_fused=True`` selects the fused
definitions regardless of size."""
from __future__ import annotations

from ..ops.loss import fused_dense_loss, fused_label_loss_supported, reference_switches_to_fused
from .contrastive import contrastive_loss


def fused_contrastive_loss(query_embeds, doc_embeds, labels, temperature=0.02, scores=None,
                           pos_qi=None, pos_di=None, pos_counts=None, loss_type="multi", scale=None,
                           num_queries=None, force_fused=False):
    Q = int(num_queries if num_queries is not None else query_embeds.shape[0])
    use_fused = (pos_qi is not None and scores is None and scale is None
                 and (force_fused or reference_switches_to_fused(Q, doc_embeds.shape[0], loss_type))
                 and isinstance(temperature, (int, float))
                 and fused_label_loss_supported(query_embeds, doc_embeds))
    if use_fused:
        return fused_dense_loss(query_embeds, doc_embeds, labels, 1.0 / float(temperature),
                                loss_type=loss_type, pos_qi=pos_qi, pos_di=pos_di,
                                pos_counts=pos_counts)
    return contrastive_loss(query_embeds, doc_embeds, labels, temperature, scores, scale=scale)
