"""Long-document encoding: chunk, batch under a token budget, pool, merge.

Same contract as the reference (lset/eval/chunked_encoder.py:16-193): documents longer than
``chunk_len`` are split into overlapping chunks, each chunk is mean-pooled, a document's embedding
is the length-weighted average of its chunk embeddings (then L2-normalised); ``last_token`` /
``cls`` pooling is only defined for single-chunk documents; tokenisation can be cached on disk;
out-of-memory batches are retried in halves; large results stream into a memmap.

The batching is different on purpose: chunks are *packed* into streams of at most
``token_budget`` tokens (no padding at all) and run through the model's packed path, instead of
padded ``(B+1)·max_len ≤ budget`` rectangles.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from ..ops.pooling import packed_pool
from ..train.data.packing import pack_sequences

DEFAULT_CHUNK_LEN = 4096
DEFAULT_OVERLAP = 128
DEFAULT_TOKEN_BUDGET = 65536  # sized for a 180 GB B200 (the reference defaults to 16384 for 16 GB)
CPU_STREAM_THRESHOLD = 50_000


def cached_tokenize(tokenize_fn: Callable[[List[str]], List[List[int]]], texts: Sequence[str],
                    cache_dir: Optional[Path] = None) -> List[List[int]]:
    """Token ids for ``texts``; with ``cache_dir`` the result is stored under a content hash."""
    if cache_dir is None:
        return tokenize_fn(list(texts))
    cache_dir = Path(cache_dir)
    cache_dir.mkdir(parents=True, exist_ok=True)
    h = hashlib.sha256()
    for t in texts:
        h.update(t.encode("utf-8", "ignore"))
        h.update(b"\0")
    f = cache_dir / f"tok_{h.hexdigest()[:24]}.json"
    if f.exists():
        return json.loads(f.read_text())
    ids = tokenize_fn(list(texts))
    f.write_text(json.dumps(ids))
    return ids


def chunk_ids(ids: List[int], chunk_len: int, overlap: int) -> List[List[int]]:
    if len(ids) <= chunk_len:
        return [ids]
    step = max(1, chunk_len - overlap)
    out = []
    for s in range(0, len(ids), step):
        out.append(ids[s:s + chunk_len])
        if s + chunk_len >= len(ids):
            break
    return out


def plan_streams(lengths: Sequence[int], budget: int) -> List[List[int]]:
    """Greedy packing of chunk indices (longest first) into streams of at most ``budget`` tokens."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    streams, cur, used = [], [], 0
    for i in order:
        n = max(1, lengths[i])
        if cur and used + n > budget:
            streams.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += n
    if cur:
        streams.append(cur)
    return streams


def encode_chunked(model, tokenize_fn, pool_fn, texts: Sequence[str], *, device, pad_id: int = 0,
                   pooling: str = "mean", normalize: bool = True, chunk_len: int = DEFAULT_CHUNK_LEN,
                   overlap: int = DEFAULT_OVERLAP, token_budget: int = DEFAULT_TOKEN_BUDGET,
                   max_pos: Optional[int] = None, out_path: Optional[str] = None,
                   dim: Optional[int] = None, tokenize_cache_dir: Optional[str] = None,
                   oom_retry_halving: bool = True, post_pooling=None) -> np.ndarray:
    if pooling not in ("mean", "last_token", "cls"):
        raise ValueError(f"unknown pooling {pooling!r}")
    encoded = cached_tokenize(tokenize_fn, texts, Path(tokenize_cache_dir) if tokenize_cache_dir else None)
    if max_pos is not None:
        encoded = [ids[:max_pos] for ids in encoded]
    if pooling != "mean" and any(len(ids) > chunk_len for ids in encoded):
        raise ValueError(f"pooling={pooling!r} is not defined across chunks; use mean pooling for "
                         f"documents longer than chunk_len={chunk_len}")
    chunks, owners = [], []
    for d, ids in enumerate(encoded):
        for c in chunk_ids(ids if ids else [pad_id], chunk_len, overlap):
            chunks.append(c)
            owners.append(d)
    N = len(texts)
    if N == 0:
        return np.zeros((0, dim or 0), dtype=np.float32)
    lens = [len(c) for c in chunks]
    device = torch.device(device)

    def run(idx: List[int]) -> torch.Tensor:
        packed = pack_sequences([chunks[i] for i in idx])
        ids = packed["input_ids"].to(device)
        cu = packed["cu_seqlens"].to(device)
        with torch.no_grad():
            hid = model(ids, position_ids=packed["position_ids"].to(device), cu_seqlens=cu,
                        max_seqlen=packed["max_seqlen"])["hidden_states"]
            return packed_pool(hid, cu, pooling, False).float()

    def run_with_retry(idx: List[int]) -> torch.Tensor:
        try:
            return run(idx)
        except torch.cuda.OutOfMemoryError:
            if not oom_retry_halving or len(idx) == 1:
                raise
            torch.cuda.empty_cache()
            half = len(idx) // 2
            return torch.cat([run_with_retry(idx[:half]), run_with_retry(idx[half:])])

    acc = None
    weight = torch.zeros(N, dtype=torch.float32, device=device)
    owners_t = torch.tensor(owners, device=device)
    lens_t = torch.tensor(lens, dtype=torch.float32, device=device)
    for stream in plan_streams(lens, token_budget):
        emb = run_with_retry(stream)
        if acc is None:
            acc = torch.zeros(N, emb.shape[1], dtype=torch.float32, device=device)
        sel = torch.tensor(stream, device=device)
        w = lens_t[sel]
        acc.index_add_(0, owners_t[sel], emb * w[:, None])
        weight.index_add_(0, owners_t[sel], w)
    out = acc / weight.clamp(min=1.0)[:, None]
    if post_pooling is not None:   # dense projection between pooling and normalisation
        with torch.no_grad():
            w_dtype = next(iter(post_pooling.buffers())).dtype
            out = post_pooling(out.to(w_dtype)).float()
    if normalize:
        out = torch.nn.functional.normalize(out, dim=-1, eps=1e-12)
    result = out.cpu().numpy().astype(np.float32)
    if out_path and N >= CPU_STREAM_THRESHOLD:
        mm = np.lib.format.open_memmap(out_path, mode="w+", dtype=np.float32, shape=result.shape)
        mm[:] = result
        mm.flush()
        return mm
    return result
