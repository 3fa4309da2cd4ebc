"""CUDA-graph capture and replay of a fixed-shape model forward.

``CUDAGraphWrapper`` covers what the reference's wrapper does (padded ``[B, S]`` inputs, forward
only; lset/train/cuda_graph.py:10-58) and, because every kernel here reads sequence boundaries
from device memory, also a packed fixed-budget stream: ``PackedCUDAGraphWrapper`` captures one
forward over ``token_budget`` tokens and ``max_sequences`` segments and replays it for any batch
produced by ``FixedBudgetPackedCollator`` (contents of ``input_ids``, ``position_ids`` and
``cu_seqlens`` change, shapes do not). ``validate_cuda_graph_config`` keeps the reference's
incompatibility rules (lset/train/cuda_graph.py:61-75).
"""
from __future__ import annotations

import torch
import torch.nn as nn


def _warm(fn, iters: int):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(iters):
            fn()
    torch.cuda.current_stream().wait_stream(side)


class CUDAGraphWrapper:
    """Padded mode: ``model(input_ids [B, S])`` with no attention mask (full rows)."""

    def __init__(self, model: nn.Module, batch_size: int, seq_length: int, device, warmup_iters: int = 3):
        self.model, self.device = model, torch.device(device)
        self.static_input_ids = torch.zeros(batch_size, seq_length, dtype=torch.long, device=self.device)
        _warm(lambda: model(self.static_input_ids), warmup_iters)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.static_output = model(self.static_input_ids)

    def forward(self, input_ids, attention_mask=None):
        self.static_input_ids.copy_(input_ids)
        self.graph.replay()
        return self.static_output

    __call__ = forward


class PackedCUDAGraphWrapper:
    """Packed fixed-budget mode. Unused trailing segments are empty (``cu`` repeats its last value),
    pad tokens belong to no segment."""

    def __init__(self, model: nn.Module, token_budget: int, max_sequences: int, device,
                 max_seqlen: int, warmup_iters: int = 3):
        self.model, self.device = model, torch.device(device)
        self.max_sequences, self.max_seqlen = max_sequences, max_seqlen
        self.ids = torch.zeros(token_budget, dtype=torch.long, device=self.device)
        self.pos = torch.zeros(token_budget, dtype=torch.long, device=self.device)
        self.cu = torch.zeros(max_sequences + 1, dtype=torch.int32, device=self.device)
        self.cu[1:] = token_budget  # one full segment for the warm-up
        run = lambda: model(self.ids, position_ids=self.pos, cu_seqlens=self.cu,  # noqa: E731
                            max_seqlen=self.max_seqlen)
        _warm(run, warmup_iters)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.static_output = run()

    def forward(self, batch: dict):
        n = batch["cu_seqlens"].numel() - 1
        if n > self.max_sequences:
            raise ValueError(f"{n} sequences exceed the captured maximum {self.max_sequences}")
        self.ids.copy_(batch["input_ids"])
        self.pos.copy_(batch["position_ids"])
        self.cu[: n + 1].copy_(batch["cu_seqlens"])
        self.cu[n + 1:] = batch["cu_seqlens"][-1]
        self.graph.replay()
        return self.static_output

    __call__ = forward


def validate_cuda_graph_config(packed: bool, use_grad_cache: bool, compile_model: bool,
                               token_budget=None) -> None:
    problems = []
    if packed and not token_budget:
        problems.append("CUDA graph with packed sequences needs a fixed token budget "
                        "(cuda_graph.token_budget); variable-length packing has dynamic shapes")
    if use_grad_cache:
        problems.append("CUDA graph is incompatible with GradCache (variable chunk shapes)")
    if compile_model:
        problems.append("CUDA graph is redundant with torch.compile")
    if problems:
        raise ValueError("CUDA graph incompatible:\n  - " + "\n  - ".join(problems))
