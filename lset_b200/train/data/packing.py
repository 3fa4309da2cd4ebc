"""Sequence packing: token lists -> one flat stream with ``cu_seqlens``
(output contract of lset/train/data/packing.py:6-21 and the fixed-budget variant of
lset/train/data/packed_collator.py:27-67)."""
from __future__ import annotations

from typing import List, Sequence

import torch


def pack_sequences(sequences: Sequence[Sequence[int]]) -> dict:
    """``{input_ids [T] int64, cu_seqlens [N+1] int32, max_seqlen int, position_ids [T] int64}``;
    positions restart at 0 for every sequence."""
    lens = [len(s) for s in sequences]
    flat = [t for s in sequences for t in s]
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    if lens:
        cu[1:] = torch.tensor(lens, dtype=torch.int64).cumsum(0).to(torch.int32)
    pos = torch.cat([torch.arange(n, dtype=torch.int64) for n in lens]) if lens else \
        torch.zeros(0, dtype=torch.int64)
    return {"input_ids": torch.tensor(flat, dtype=torch.int64), "cu_seqlens": cu,
            "max_seqlen": max(lens) if lens else 0, "position_ids": pos}


def pack_fixed_budget(sequences: Sequence[Sequence[int]], token_budget: int, pad_token_id: int = 0) -> dict:
    """Pack greedily until ``token_budget``: empty sequences and sequences that do not fit are
    skipped, and the stream is padded at the end to exactly ``token_budget`` tokens (pad tokens
    belong to no sequence, position 0) — fixed shapes for CUDA-graph replay. ``num_sequences``
    counts the packed sequences."""
    kept: List[Sequence[int]] = []
    used = 0
    for s in sequences:
        if len(s) == 0 or used + len(s) > token_budget:
            continue
        kept.append(s)
        used += len(s)
    out = pack_sequences(kept)
    pad = token_budget - used
    if pad > 0:
        out["input_ids"] = torch.cat([out["input_ids"], torch.full((pad,), pad_token_id, dtype=torch.int64)])
        out["position_ids"] = torch.cat([out["position_ids"], torch.zeros(pad, dtype=torch.int64)])
    out["max_seqlen"] = max(out["max_seqlen"], 1)
    out["num_sequences"] = len(kept)
    return out


_pack_fixed_budget = pack_fixed_budget
