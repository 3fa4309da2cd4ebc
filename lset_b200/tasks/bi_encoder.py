"""Bi-encoder contrastive task: encode queries and documents, pool, gather negatives, loss.

Same call surface as the reference task (lset/tasks/bi_encoder.py:34-146): ``encode(model, batch)``
and ``forward(model, query_batch, doc_batch, neg_batch=None, labels=None, scores=None, pos_qi=None,
pos_di=None, pos_counts=None) -> {"loss", "query_embeds", "doc_embeds"}``. Two deliberate
differences in how the work is done:

* packed query / document / negative batches are concatenated into ONE token stream and encoded in
  a single forward (every layer's weights are touched once instead of two or three times);
* under data parallelism each rank scores only its own query rows against the globally gathered
  documents, and document gradients return to their owners through a reduce-scatter. The loss is
  normalised by the *global* number of queries, so the value (after summing over ranks) and the
  data-parallel-averaged parameter gradient equal the reference's, which evaluates the whole
  global matrix redundantly on every rank.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..dist.gather import gather_for_local_rows
from ..losses.base import LogitScale
from ..losses.contrastive import contrastive_loss
from ..losses.fused_contrastive import fused_contrastive_loss
from ..losses.infonce import infonce_loss
from ..losses.matryoshka import matryoshka_loss
from ..ops.pooling import packed_pool, pool


def concat_packed(batches):
    """Concatenate packed batches (dicts with input_ids, position_ids, cu_seqlens, max_seqlen) into
    one stream. Returns ``(merged, counts)`` where counts are the sequences per input batch."""
    ids = torch.cat([b["input_ids"] for b in batches])
    pos = torch.cat([b["position_ids"] for b in batches])
    cus, counts, off = [], [], 0
    for i, b in enumerate(batches):
        cu = b["cu_seqlens"].to(torch.int32)
        cus.append((cu if i == 0 else cu[1:]) + off)
        off += int(b["input_ids"].shape[0])
        counts.append(cu.numel() - 1)
    merged = {"input_ids": ids, "position_ids": pos, "cu_seqlens": torch.cat(cus),
              "max_seqlen": max(int(b["max_seqlen"]) for b in batches)}
    return merged, counts


class BiEncoderTask(nn.Module):
    def __init__(self, pooling: str = "last_token", normalize: bool = True,
                 temperature: float = 0.02, matryoshka_dims=None, top_k: Optional[int] = None,
                 learnable_scale: bool = False, max_scale: float = 100.0, cascade: bool = False,
                 cascade_d_small: int = 64, cascade_K_prime: int = 256, dp_group=None,
                 joint_encode: bool = True):
        super().__init__()
        self.pooling = pooling
        self.normalize = normalize
        self.temperature = temperature
        self.matryoshka_dims = matryoshka_dims
        self.top_k = top_k
        self.dp_group = dp_group
        self.joint_encode = joint_encode
        # optional module applied to the pooled embedding before normalisation (``ModelSpec.
        # post_pooling_fn``: EmbeddingGemma's dense projection); frozen, not part of the state dict
        self.__dict__["post_pooling"] = None
        self.logit_scale = (LogitScale.from_temperature(temperature, learnable=True,
                                                        max_scale=max_scale)
                            if learnable_scale else None)

    def set_post_pooling(self, module) -> None:
        """Install (or clear) the post-pooling projection without registering it as a submodule."""
        self.__dict__["post_pooling"] = module

    # ------------------------------------------------------------------ encoding
    def _norm_flag(self):
        return self.normalize and self.matryoshka_dims is None

    def encode(self, model: nn.Module, batch: dict) -> torch.Tensor:
        proj = self.post_pooling
        norm = self._norm_flag() and proj is None
        if "cu_seqlens" in batch:
            out = model.forward_packed(batch["input_ids"], batch["position_ids"],
                                       batch["cu_seqlens"], batch["max_seqlen"])
            emb = packed_pool(out["hidden_states"], batch["cu_seqlens"], self.pooling, norm)
        else:
            out = model(batch["input_ids"], batch["attention_mask"])
            emb = pool(out["hidden_states"], batch["attention_mask"], self.pooling, norm)
        if proj is not None:
            from ..ops.pooling import normalize

            emb = proj(emb)
            if self._norm_flag():
                emb = normalize(emb)
        return emb

    def encode_many(self, model: nn.Module, batches):
        """Embeddings for several batches; packed ones share a single forward pass."""
        batches = [b for b in batches if b is not None]
        if self.joint_encode and len(batches) > 1 and all("cu_seqlens" in b for b in batches):
            merged, counts = concat_packed(batches)
            emb = self.encode(model, merged)
            return list(torch.split(emb, counts, dim=0))
        return [self.encode(model, b) for b in batches]

    # ------------------------------------------------------------------ loss
    def _dp(self):
        if dist.is_available() and dist.is_initialized():
            return dist.get_world_size(self.dp_group), dist.get_rank(self.dp_group)
        return 1, 0

    def current_temperature(self):
        if self.logit_scale is not None:
            return 1.0 / self.logit_scale()
        return self.temperature

    def loss_from_embeddings(self, q_emb, d_emb, n_emb=None, labels=None, scores=None,
                             pos_qi=None, pos_di=None, pos_counts=None):
        """Loss for local query rows against globally gathered documents (+ negatives).
        Returns the rank's share of the global mean (the shares sum to the global loss)."""
        W, rank = self._dp()
        Bq, Bd = q_emb.shape[0], d_emb.shape[0]
        if (W > 1 and labels is None and self.matryoshka_dims is None
                and self.top_k is None and self.logit_scale is None and Bq == Bd):
            from ..dist import xrank_loss

            # Hard negatives ride along: every rank publishes [its documents; its negatives] as one
            # block. The softmax runs over all columns whatever their order, and the positive of
            # local query i is still row i of this rank's block.
            local_docs = d_emb if n_emb is None else torch.cat([d_emb, n_emb], dim=0)
            if xrank_loss.supported(q_emb, local_docs, self.dp_group):
                # gather, similarity GEMM, logsumexp and the dK reduce-scatter fused over NVLink
                return xrank_loss.cross_rank_infonce(q_emb, local_docs, self.temperature,
                                                     self.dp_group)
        docs = gather_for_local_rows(d_emb, self.dp_group)
        if n_emb is not None:
            docs = torch.cat([docs, gather_for_local_rows(n_emb, self.dp_group)], dim=0)
        temperature = self.current_temperature()
        if labels is not None:
            labels = labels.to(q_emb.device)
            Kn = docs.shape[0]
            if labels.shape[1] != Kn:
                # local [Bq, Bd(+negs)] block placed at this rank's document columns
                full = torch.zeros(Bq, Kn, dtype=labels.dtype, device=labels.device)
                full[:, rank * Bd:(rank + 1) * Bd] = labels[:, :Bd]
                if labels.shape[1] > Bd and n_emb is not None:
                    Bn = n_emb.shape[0]
                    full[:, W * Bd + rank * Bn: W * Bd + (rank + 1) * Bn] = labels[:, Bd:]
                labels_full = full
                s_full = None
                if scores is not None:
                    s_full = torch.full((Bq, Kn), float("-inf"), device=q_emb.device)
                    s_full[:, rank * Bd:(rank + 1) * Bd] = scores.to(q_emb.device)[:, :Bd]
            else:
                labels_full, s_full = labels, (scores.to(q_emb.device) if scores is not None else None)
            if self.matryoshka_dims:
                local = matryoshka_loss(q_emb, docs, self.matryoshka_dims, temperature, labels_full)
            elif isinstance(temperature, (int, float)):
                pdi = None
                if pos_qi is not None and pos_di is not None:
                    # local document indices -> columns of the gathered [docs | negatives] matrix
                    pdi = pos_di.to(q_emb.device).long()
                    if W > 1:
                        Bn = n_emb.shape[0] if n_emb is not None else 0
                        pdi = torch.where(pdi < Bd, pdi + rank * Bd, pdi - Bd + W * Bd + rank * Bn)
                local = fused_contrastive_loss(
                    q_emb, docs, labels_full, temperature, s_full,
                    pos_qi=pos_qi.to(q_emb.device) if pos_qi is not None and pdi is not None else None,
                    pos_di=pdi, pos_counts=pos_counts, num_queries=W * Bq)
            else:
                local = contrastive_loss(q_emb, docs, labels_full, temperature, s_full)
            return local / W if W > 1 else local
        if self.matryoshka_dims is not None:
            local = matryoshka_loss(q_emb, docs, self.matryoshka_dims, temperature,
                                    target_offset=rank * Bd)
        else:
            local = infonce_loss(q_emb, docs, temperature, self.top_k, target_offset=rank * Bd)
        return local / W if W > 1 else local

    def forward(self, model: nn.Module, query_batch: dict, doc_batch: dict,
                neg_batch: Optional[dict] = None, labels=None, scores=None, pos_qi=None,
                pos_di=None, pos_counts=None) -> dict:
        embs = self.encode_many(model, [query_batch, doc_batch, neg_batch])
        q_emb, d_emb = embs[0], embs[1]
        n_emb = embs[2] if len(embs) > 2 else None
        loss = self.loss_from_embeddings(q_emb, d_emb, n_emb, labels, scores, pos_qi, pos_di,
                                         pos_counts)
        return {"loss": loss, "query_embeds": q_emb.detach(), "doc_embeds": d_emb.detach()}


def global_loss_value(local_loss: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the per-rank loss shares = the global mean loss (for logging)."""
    v = local_loss.detach().clone()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(v, op=dist.ReduceOp.SUM, group=group)
    return v
