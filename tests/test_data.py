"""Packing, collators and dataset formats."""
import json

import torch

from lset_b200.train.data.collator import (EmbeddingCollator, FixedBudgetPackedCollator,
                                           FixedLengthCollator, LeftPadCollator, PackedCollator,
                                           RightPadCollator)
from lset_b200.train.data.dataset import EmbeddingDataset, SyntheticPairDataset, detect_format
from lset_b200.train.data.packing import pack_fixed_budget, pack_sequences


def _tok(ids):
    return {"input_ids": list(ids), "attention_mask": [1] * len(ids)}


def test_pack_sequences():
    out = pack_sequences([[1, 2, 3], [4], [5, 6]])
    assert out["input_ids"].tolist() == [1, 2, 3, 4, 5, 6] and out["input_ids"].dtype == torch.int64
    assert out["cu_seqlens"].tolist() == [0, 3, 4, 6] and out["cu_seqlens"].dtype == torch.int32
    assert out["position_ids"].tolist() == [0, 1, 2, 0, 0, 1] and out["max_seqlen"] == 3


def test_fixed_budget_skips_and_pads():
    out = pack_fixed_budget([[1, 2, 3], [4, 5, 6, 7, 8], [], [9, 10]], token_budget=6, pad_token_id=0)
    assert out["input_ids"].tolist() == [1, 2, 3, 9, 10, 0] and out["num_sequences"] == 2
    assert out["cu_seqlens"].tolist() == [0, 3, 5] and out["position_ids"].tolist() == [0, 1, 2, 0, 1, 0]


def test_pad_collators():
    batch = [{"query": _tok([1, 2]), "positive": _tok([3, 4, 5]), "negative": _tok([6])},
             {"query": _tok([7]), "positive": _tok([8]), "negative": _tok([9, 10])}]
    left = LeftPadCollator(0)(batch)
    assert left["query"]["input_ids"].tolist() == [[1, 2], [0, 7]]
    assert left["query"]["attention_mask"].tolist() == [[1, 1], [0, 1]] and "neg" in left
    right = RightPadCollator(99)(batch)
    assert right["doc"]["input_ids"].tolist() == [[3, 4, 5], [8, 99, 99]]
    fixed = FixedLengthCollator(0, 4)(batch)
    assert fixed["doc"]["input_ids"].shape == (2, 4) and fixed["doc"]["input_ids"][1].tolist() == [0, 0, 0, 8]
    packed = PackedCollator()(batch)
    assert packed["doc"]["cu_seqlens"].tolist() == [0, 3, 4]
    fb = FixedBudgetPackedCollator(8)(batch)
    assert fb["query"]["input_ids"].numel() == 8 and fb["query"]["num_sequences"] == 2


def test_collators_flatten_a_list_of_hard_negatives():
    """``"negatives"`` (a list per sample) lands in ``"neg"`` sample by sample, as one
    ``"negative"`` per sample does."""
    batch = [{"query": _tok([1]), "positive": _tok([2]), "negatives": [_tok([3, 4]), _tok([5])]},
             {"query": _tok([6]), "positive": _tok([7]), "negatives": [_tok([8]), _tok([9, 10, 11])]}]
    packed = PackedCollator()(batch)
    assert packed["neg"]["input_ids"].tolist() == [3, 4, 5, 8, 9, 10, 11]
    assert packed["neg"]["cu_seqlens"].tolist() == [0, 2, 3, 4, 7]
    right = RightPadCollator(0)(batch)
    assert right["neg"]["input_ids"].tolist() == [[3, 4, 0], [5, 0, 0], [8, 0, 0], [9, 10, 11]]
    ds = SyntheticPairDataset(4, 50, (2, 3), (3, 5), num_negatives=3, seed=1)
    out = PackedCollator()([ds[i] for i in range(4)])
    assert out["neg"]["cu_seqlens"].numel() == 4 * 3 + 1


class _FakeTok:
    class _E:
        def __init__(self, ids):
            self.ids = ids

    def encode(self, text):
        return self._E([len(w) for w in text.split()])


def test_embedding_collator_labels_and_sorting():
    batch = [{"query": "a bb", "positives": ["p one", "p two"], "negatives": ["n"], "scores": None},
             {"query": "a much longer query here", "positives": ["q"], "negatives": [], "scores": None}]
    out = EmbeddingCollator(_FakeTok(), max_length=3, packed=True, length_sorted=True)(batch)
    assert out["labels"].shape == (2, 4)
    assert out["labels"].tolist() == [[1, 0, 0, 0], [0, 1, 1, 0]]  # longest query first
    assert out["pos_qi"].tolist() == [0, 1, 1] and out["pos_di"].tolist() == [0, 1, 2]
    assert out["pos_counts"].tolist() == [1, 2]
    assert out["query"]["cu_seqlens"].tolist() == [0, 3, 5]  # truncated to max_length
    padded = EmbeddingCollator(_FakeTok(), packed=False)(batch)
    assert padded["query"]["attention_mask"].tolist() == [[0, 0, 0, 1, 1], [1, 1, 1, 1, 1]]


def test_embedding_collator_scored():
    batch = [{"query": "q", "positives": ["a"], "negatives": ["b"], "scores": [2.0, 0.0],
              "all_documents": ["a", "b"]}]
    out = EmbeddingCollator(_FakeTok())(batch)
    assert out["labels"].tolist() == [[1, 0]] and out["scores"].tolist() == [[2.0, 0.0]]


def test_dataset_formats(tmp_path):
    recs = {
        "pair": {"query": "q", "positive": "p"},
        "triplet": {"query": "q", "positive": "p", "negatives": ["n1", "n2", "n3"]},
        "multi": {"query": "q", "positives": ["p1", "p2"], "negatives": ["n"]},
        "scored": {"query": "q", "documents": [{"text": "a", "score": 1}, {"text": "b", "score": 0}]},
    }
    for fmt, rec in recs.items():
        assert detect_format(rec) == fmt
        f = tmp_path / f"{fmt}.jsonl"
        f.write_text(json.dumps(rec) + "\n\n")
        ds = EmbeddingDataset(f, tokenizer=None, num_hard_negatives=2)
        assert ds.format == fmt and len(ds) == 1
        item = ds[0]
        assert item["query"] == "q"
        if fmt == "triplet":
            assert item["negatives"] == ["n1", "n2"]
        if fmt == "scored":
            assert item["scores"] == [1, 0] and item["all_documents"] == ["a", "b"]
    j = tmp_path / "list.json"
    j.write_text(json.dumps([recs["pair"], recs["pair"]]))
    assert len(EmbeddingDataset(j)) == 2


def test_synthetic_dataset_is_deterministic():
    a, b = SyntheticPairDataset(4, 100, seed=3), SyntheticPairDataset(4, 100, seed=3)
    assert a[2] == b[2] and 16 <= len(a[0]["query"]["input_ids"]) <= 64
