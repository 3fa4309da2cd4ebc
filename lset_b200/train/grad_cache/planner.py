"""Minibatch planning and feature slicing for GradCache.

A feature dict is either padded (``input_ids [B,S]``, ``attention_mask``) or packed
(``input_ids [T]``, ``cu_seqlens``, ``position_ids``, ``max_seqlen``). Plans are lists of
``(begin, end)`` sequence ranges: fixed size, or greedy under a token budget for packed features
(planning rules of lset/train/grad_cache/minibatch_backward.py:17-66; slicing of
lset/train/grad_cache/wrapper.py:34-64).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

Range = Tuple[int, int]


def num_units(feature: dict) -> int:
    if "cu_seqlens" in feature:
        return int(feature["cu_seqlens"].shape[0]) - 1
    return int(feature["input_ids"].shape[0])


def sequence_lengths(feature: dict) -> List[int]:
    if "seq_lengths" in feature:
        sl = feature["seq_lengths"]
        return sl.tolist() if torch.is_tensor(sl) else list(sl)
    cu = feature["cu_seqlens"]
    return (cu[1:] - cu[:-1]).tolist()


def fixed_size_plan(n: int, size: int) -> List[Range]:
    size = max(1, int(size))
    return [(b, min(b + size, n)) for b in range(0, n, size)]


def token_budget_plan(lengths: Sequence[int], budget: int) -> List[Range]:
    """Greedy: close the current chunk when the next sequence would overflow the budget (a single
    sequence longer than the budget still gets a chunk of its own)."""
    plan, begin, used = [], 0, 0
    for i, n in enumerate(lengths):
        if used + n > budget and used > 0:
            plan.append((begin, i))
            begin, used = i, 0
        used += int(n)
    if begin < len(lengths):
        plan.append((begin, len(lengths)))
    return plan


def plan_minibatches(feature: dict, mini_batch_size: Optional[int],
                     token_budget: Optional[int] = None) -> List[Range]:
    if "cu_seqlens" in feature and token_budget is not None:
        return token_budget_plan(sequence_lengths(feature), token_budget)
    return fixed_size_plan(num_units(feature), mini_batch_size or num_units(feature) or 1)


def slice_feature(feature: dict, begin: int, end: int, lengths: Optional[Sequence[int]] = None) -> dict:
    """Sub-batch with sequences ``[begin, end)``. Padded slices drop columns that are padding in
    every kept row (right padding trimmed on the right, left padding on the left)."""
    if "cu_seqlens" in feature:
        cu = feature["cu_seqlens"]
        if lengths is None:
            lengths = sequence_lengths(feature)
        t0 = int(sum(lengths[:begin]))
        t1 = t0 + int(sum(lengths[begin:end]))
        out = {"input_ids": feature["input_ids"][t0:t1],
               "position_ids": feature["position_ids"][t0:t1],
               "cu_seqlens": (cu[begin:end + 1] - cu[begin]).to(cu.dtype),
               "max_seqlen": max([int(x) for x in lengths[begin:end]] or [1])}
        return out
    ids, mask = feature["input_ids"][begin:end], feature["attention_mask"][begin:end]
    cols = mask.any(dim=0)
    if bool(cols.any()) and not bool(cols.all()):
        nz = torch.nonzero(cols).flatten()
        lo, hi = int(nz[0]), int(nz[-1]) + 1
        ids, mask = ids[:, lo:hi], mask[:, lo:hi]
    out = {"input_ids": ids, "attention_mask": mask}
    for k, v in feature.items():
        if k not in out and torch.is_tensor(v) and v.shape[:1] == feature["input_ids"].shape[:1]:
            out[k] = v[begin:end]
    return out
