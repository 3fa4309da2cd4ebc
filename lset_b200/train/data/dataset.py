"""Text datasets for contrastive training.

``EmbeddingDataset`` reads a JSONL file or a JSON list and detects the record format from the
first record: ``scored`` (``documents: [{text, score}]``), ``multi`` (``positives: [...]``),
``triplet`` (``positive`` + ``negatives``) or ``pair`` (``query`` + ``positive``). Items are *text*
dicts ``{query, positives, negatives, scores[, all_documents]}``; tokenisation happens in the
collator (record contract of lset/train/data/dataset.py:11-111).

``SyntheticPairDataset`` yields pre-tokenised random pairs of configurable length ranges; the
benchmarks and smoke tests use it (no files or tokenizer needed).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch
from torch.utils.data import Dataset


def read_records(path) -> list:
    path = Path(path)
    if path.suffix == ".jsonl":
        with open(path) as fh:
            return [json.loads(line) for line in fh if line.strip()]
    with open(path) as fh:
        data = json.load(fh)
    if not isinstance(data, list):
        raise ValueError("JSON file must contain a list of samples")
    return data


def detect_format(record: dict) -> str:
    for key, fmt in (("documents", "scored"), ("positives", "multi"), ("negatives", "triplet")):
        if key in record:
            return fmt
    return "pair"


class EmbeddingDataset(Dataset):
    def __init__(self, data_path, tokenizer=None, max_length: int = 512, template=None,
                 num_hard_negatives: Optional[int] = 0):
        self.tokenizer = tokenizer
        self.max_length = max_length
        self.template = template
        self.num_hard_negatives = num_hard_negatives or 0
        self.samples = read_records(data_path)
        self.format = detect_format(self.samples[0]) if self.samples else "pair"

    def __len__(self):
        return len(self.samples)

    def _q(self, text: str) -> str:
        return self.template.format_query(text) if self.template is not None else text

    def _d(self, text: str) -> str:
        return self.template.format_document(text) if self.template is not None else text

    def __getitem__(self, idx):
        rec = self.samples[idx]
        query = self._q(rec["query"])
        if self.format == "scored":
            docs = rec["documents"]
            texts = [self._d(d["text"]) for d in docs]
            pos = [t for t, d in zip(texts, docs) if d["score"] > 0]
            neg = [t for t, d in zip(texts, docs) if d["score"] == 0]
            return {"query": query, "positives": pos or texts[:1], "negatives": neg,
                    "scores": [d["score"] for d in docs], "all_documents": texts}
        if self.format == "multi":
            pos = [self._d(t) for t in rec["positives"]]
        else:
            pos = [self._d(rec["positive"])]
        neg = [self._d(t) for t in rec.get("negatives", [])] if self.format != "pair" else []
        if self.num_hard_negatives > 0 and neg:
            neg = neg[: self.num_hard_negatives]
        return {"query": query, "positives": pos, "negatives": neg, "scores": None}


class SyntheticPairDataset(Dataset):
    """Random pre-tokenised (query, positive[, negatives]) samples, deterministic per index."""

    def __init__(self, num_samples: int, vocab_size: int, query_len=(16, 64), doc_len=(128, 512),
                 num_negatives: int = 0, seed: int = 0, min_token_id: int = 0):
        self.n, self.vocab, self.seed = num_samples, vocab_size, seed
        self.query_len, self.doc_len, self.num_negatives = query_len, doc_len, num_negatives
        self.min_token_id = min_token_id

    def __len__(self):
        return self.n

    def _seq(self, gen, lo_hi):
        n = int(torch.randint(lo_hi[0], lo_hi[1] + 1, (1,), generator=gen))
        ids = torch.randint(self.min_token_id, self.vocab, (n,), generator=gen).tolist()
        return {"input_ids": ids, "attention_mask": [1] * n}

    def __getitem__(self, idx):
        gen = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        item = {"query": self._seq(gen, self.query_len), "positive": self._seq(gen, self.doc_len)}
        if self.num_negatives == 1:
            item["negative"] = self._seq(gen, self.doc_len)
        elif self.num_negatives > 1:
            item["negatives"] = [self._seq(gen, self.doc_len) for _ in range(self.num_negatives)]
        return item
