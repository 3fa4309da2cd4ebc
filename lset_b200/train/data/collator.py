"""Batch collators.

Pre-tokenised samples ``{"query": {...}, "positive": {...}[, "negative": {...}]}`` go through
``LeftPadCollator`` (last-token pooling), ``RightPadCollator`` (mean / CLS pooling),
``FixedLengthCollator`` (always ``max_seq_length`` wide, left padded), ``PackedCollator`` or
``FixedBudgetPackedCollator``; text samples from ``EmbeddingDataset`` go through
``EmbeddingCollator``, which tokenises, optionally sorts the batch by query length, flattens the
documents (positives then negatives per sample) and builds the ``[Q, K]`` label matrix, the
positive-pair index lists and, for scored data, the teacher-score matrix. Output contracts follow
lset/train/data/collator.py:8-238 and lset/train/data/packed_collator.py:8-90.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .packing import pack_fixed_budget, pack_sequences


def pad_batch(sequences: Sequence[dict], pad_token_id: int, side: str = "left",
              width: Optional[int] = None) -> dict:
    """Pad ``{"input_ids", "attention_mask"}`` samples to a rectangle; ``width`` fixes the size
    (longer samples are truncated)."""
    seqs = [(s["input_ids"], s["attention_mask"]) for s in sequences]
    if width is not None:
        seqs = [(i[:width], m[:width]) for i, m in seqs]
    W = width if width is not None else max((len(i) for i, _ in seqs), default=0)
    ids = torch.full((len(seqs), W), pad_token_id, dtype=torch.long)
    mask = torch.zeros((len(seqs), W), dtype=torch.long)
    for r, (i, m) in enumerate(seqs):
        n = len(i)
        if n == 0:
            continue
        sl = slice(W - n, W) if side == "left" else slice(0, n)
        ids[r, sl] = torch.tensor(i, dtype=torch.long)
        mask[r, sl] = torch.tensor(m, dtype=torch.long)
    return {"input_ids": ids, "attention_mask": mask}


class _TripleCollator:
    """query / positive / optional negative(s) -> ``{"query", "doc"[, "neg"]}``. A sample may carry
    one hard negative (``"negative"``) or a list of them (``"negatives"``, flattened sample by
    sample: negative j of sample i is row ``i * n + j``)."""

    def _batch(self, seqs: List[dict]) -> dict:  # pragma: no cover - overridden
        raise NotImplementedError

    def __call__(self, batch: List[dict]) -> dict:
        out = {"query": self._batch([s["query"] for s in batch]),
               "doc": self._batch([s["positive"] for s in batch])}
        if "negative" in batch[0]:
            out["neg"] = self._batch([s["negative"] for s in batch])
        elif batch[0].get("negatives"):
            out["neg"] = self._batch([n for s in batch for n in s["negatives"]])
        return out


class LeftPadCollator(_TripleCollator):
    def __init__(self, pad_token_id: int):
        self.pad_token_id = pad_token_id

    def _batch(self, seqs):
        return pad_batch(seqs, self.pad_token_id, "left")


class RightPadCollator(_TripleCollator):
    def __init__(self, pad_token_id: int):
        self.pad_token_id = pad_token_id

    def _batch(self, seqs):
        return pad_batch(seqs, self.pad_token_id, "right")


class FixedLengthCollator(_TripleCollator):
    def __init__(self, pad_token_id: int, max_seq_length: int):
        self.pad_token_id, self.max_seq_length = pad_token_id, max_seq_length

    def _batch(self, seqs):
        return pad_batch(seqs, self.pad_token_id, "left", width=self.max_seq_length)


class PackedCollator(_TripleCollator):
    def _batch(self, seqs):
        return pack_sequences([s["input_ids"] for s in seqs])


class FixedBudgetPackedCollator(_TripleCollator):
    def __init__(self, token_budget: int, pad_token_id: int = 0):
        self.token_budget, self.pad_token_id = token_budget, pad_token_id

    def _batch(self, seqs):
        return pack_fixed_budget([s["input_ids"] for s in seqs], self.token_budget, self.pad_token_id)


class EmbeddingCollator:
    """Text samples -> tokenised query / document batches plus label (and score) matrices."""

    def __init__(self, tokenizer, max_length: int = 512, packed: bool = False,
                 length_sorted: bool = False, padding_side: str = "left", pad_token_id: int = 0):
        self.tokenizer = tokenizer
        self.max_length = max_length
        self.packed = packed
        self.length_sorted = length_sorted
        self.padding_side = padding_side
        self.pad_token_id = pad_token_id

    def _tokenize(self, text: str) -> dict:
        ids = self.tokenizer.encode(text).ids[: self.max_length]
        return {"input_ids": ids, "attention_mask": [1] * len(ids)}

    def _collate(self, seqs: List[dict]) -> dict:
        if self.packed:
            return pack_sequences([s["input_ids"] for s in seqs])
        return pad_batch(seqs, self.pad_token_id, self.padding_side)

    @staticmethod
    def _docs_of(sample: dict, scored: bool):
        if scored:
            docs = sample.get("all_documents")
            if docs is None:
                docs = list(sample["positives"]) + list(sample.get("negatives", []))
            return docs, [float(s) > 0 for s in sample["scores"]]
        pos, neg = list(sample["positives"]), list(sample.get("negatives", []))
        return pos + neg, [True] * len(pos) + [False] * len(neg)

    def __call__(self, batch: List[dict]) -> dict:
        if self.length_sorted:
            batch = sorted(batch, key=lambda s: len(s["query"]), reverse=True)
        scored = batch[0].get("scores") is not None
        queries = [self._tokenize(s["query"]) for s in batch]
        docs: List[dict] = []
        spans, flags = [], []
        for s in batch:
            texts, is_pos = self._docs_of(s, scored)
            spans.append((len(docs), len(texts)))
            flags.append(is_pos)
            docs.extend(self._tokenize(t) for t in texts)
        Q, K = len(batch), len(docs)
        labels = torch.zeros(Q, K)
        qi, di, counts = [], [], []
        for i, ((start, n), is_pos) in enumerate(zip(spans, flags)):
            cols = [start + j for j, p in enumerate(is_pos[:n]) if p]
            labels[i, cols] = 1.0
            qi.extend([i] * len(cols))
            di.extend(cols)
            counts.append(len(cols))
        out = {"query": self._collate(queries), "doc": self._collate(docs), "labels": labels,
               "pos_qi": torch.tensor(qi, dtype=torch.long),
               "pos_di": torch.tensor(di, dtype=torch.long),
               "pos_counts": torch.tensor(counts, dtype=torch.long)}
        if scored:
            sc = torch.full((Q, K), float("-inf"))
            for i, ((start, n), s) in enumerate(zip(spans, batch)):
                vals = torch.tensor([float(v) for v in s["scores"]][:n])
                sc[i, start:start + len(vals)] = vals
            out["scores"] = sc
        return out
