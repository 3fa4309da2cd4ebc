"""Tensor parallelism over a process group.

``apply_tp(model, tp_group, plan)`` shards, in place, every linear layer named by the plan
(``lset_b200.models.parallel_plan``): ``colwise`` layers keep a slice of the output features,
``rowwise`` layers a slice of the input features. Fused ``qkv_proj`` / ``gate_up_proj`` weights are
split section by section so every rank holds whole heads of q, k and v (resp. matching gate / up
columns). Activations follow the Megatron scheme: the input of a column-parallel layer is
replicated (its gradient is all-reduced), the output of a row-parallel layer is all-reduced.
Modules keep their names and ``weight`` attributes, the attention / MLP code derives local head
counts from the weight shapes (as in lset/models/decoder/qwen3/attention.py:92-100), and sharded
parameters are tagged ``_tp_sharded`` so the optimizer can form the correct global gradient norm.

Counterpart of ``parallelize_module`` + the Colwise/Rowwise plans of the reference
(lset/distributed/tp.py:9-11, lset/models/decoder/qwen3/parallel_plan.py:22-50).
"""
from __future__ import annotations

import fnmatch
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


class _CopyToTP(torch.autograd.Function):
    """Identity forward; all-reduce of the gradient in backward (input of column-parallel layers)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward; identity backward (output of row-parallel layers)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def _section_sizes(name: str, module: nn.Module, parent: nn.Module) -> Optional[List[int]]:
    """Row sections of a fused projection weight, or None for a plain layer."""
    leaf = name.rsplit(".", 1)[-1]
    out = module.weight.shape[0]
    if leaf == "qkv_proj":
        hd = getattr(parent, "head_dim")
        nq = getattr(parent, "num_heads") * hd
        nkv = getattr(parent, "num_kv_heads", getattr(parent, "num_heads")) * hd
        return [nq, nkv, nkv] if nq + 2 * nkv == out else [out // 3] * 3
    if leaf == "gate_up_proj":
        return [out // 2, out // 2]
    return None


def _shard_rows(t: torch.Tensor, sections: Optional[List[int]], rank: int, world: int) -> torch.Tensor:
    if sections is None:
        sections = [t.shape[0]]
    parts, start = [], 0
    for n in sections:
        if n % world:
            raise ValueError(f"cannot split {n} output features over {world} tensor-parallel ranks")
        per = n // world
        parts.append(t[start + rank * per: start + (rank + 1) * per])
        start += n
    return torch.cat(parts, dim=0).contiguous()


def _wrap_forward_sp(module: nn.Module, kind: str, st) -> None:
    """Sequence-parallel variant: the collectives are part of the (fused) linear ops."""
    from . import tp_fused

    if kind == "colwise":
        def forward(x):
            return tp_fused.ag_linear(x, module.weight, module.bias, st)
    else:
        def forward(x):
            return tp_fused.linear_rs(x, module.weight, module.bias, st)

    module.forward = forward
    module._tp_kind = kind
    module._sp_state = st      # the block runner drives the same buffers when it takes the block


def _wrap_forward(module: nn.Module, kind: str, group) -> None:
    inner = module.forward

    if kind == "colwise":
        def forward(x):
            return inner(_CopyToTP.apply(x, group))
    else:
        bias = module.bias

        def forward(x):
            # the bias of a row-parallel layer is added once, after the reduction
            if bias is not None:
                module.bias = None
                try:
                    y = inner(x)
                finally:
                    module.bias = bias
                return _ReduceFromTP.apply(y, group) + bias
            return _ReduceFromTP.apply(inner(x), group)

    module.forward = forward
    module._tp_kind = kind


def apply_tp(model: nn.Module, tp_group, plan: Dict[str, str],
             sequence_parallel: Optional[bool] = None) -> nn.Module:
    """``sequence_parallel`` (default: on when the plan marks the norms ``"sequence"``) shards the
    residual stream by tokens between the blocks and swaps the all-reduces for all-gather /
    reduce-scatter pairs fused into the GEMMs (``lset_b200.dist.tp_fused``)."""
    world, rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
    if world == 1:
        return model
    cfg = getattr(model, "config", None)
    for field in ("num_attention_heads", "num_key_value_heads"):
        heads = getattr(cfg, field, None)
        if isinstance(heads, int) and heads % world:
            raise ValueError(f"{field}={heads} cannot be split over {world} tensor-parallel ranks "
                             f"(whole attention heads stay on one rank)")
    if sequence_parallel is None:
        sequence_parallel = any(v == "sequence" for v in plan.values())
    sp_state = None
    if sequence_parallel:
        if not hasattr(model, "_sp"):
            raise ValueError(f"{type(model).__name__} has no sequence-parallel forward")
        if any(isinstance(m, nn.Linear) and n.rsplit(".", 1)[-1] in ("lora_A", "lora_B")
               for n, m in model.named_modules()):
            raise ValueError("sequence parallelism is not combined with LoRA adapters")
        from .tp_fused import SPState

        sp_state = SPState(tp_group)
    for name, module in list(model.named_modules()):
        kind = next((k for pat, k in plan.items() if fnmatch.fnmatchcase(name, pat)), None)
        if kind not in ("colwise", "rowwise") or not isinstance(module, nn.Linear):
            continue
        parent_name = name.rsplit(".", 1)[0] if "." in name else ""
        # LoRA wrappers: "....q_proj.base_linear" -> sections are decided by the attention module
        owner_name = parent_name
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("base_linear", "lora_A", "lora_B"):
            owner_name = parent_name.rsplit(".", 1)[0] if "." in parent_name else ""
        owner = model.get_submodule(owner_name) if owner_name else model
        w = module.weight.data
        if kind == "colwise":
            target_name = parent_name if leaf in ("base_linear", "lora_B") else name
            sections = _section_sizes(target_name, module, owner)
            module.weight.data = _shard_rows(w, sections, rank, world)
            module.weight._tp_meta = ("rows", sections or [w.shape[0]])
            if module.bias is not None:
                module.bias.data = _shard_rows(module.bias.data, sections, rank, world)
                module.bias._tp_sharded = True
                module.bias._tp_meta = ("rows", sections or [w.shape[0]])
            module.out_features = module.weight.shape[0]
        else:
            if w.shape[1] % world:
                raise ValueError(f"{name}: {w.shape[1]} input features not divisible by tp={world}")
            per = w.shape[1] // world
            module.weight.data = w[:, rank * per:(rank + 1) * per].contiguous()
            module.weight._tp_meta = ("cols", [w.shape[1]])
            module.in_features = per
        module.weight._tp_sharded = True
        # lora_A of a colwise target / lora_B of a rowwise target stay replicated and un-hooked;
        # the hooks go on the layers that actually change the activation layout.
        if leaf == "lora_B" and kind == "colwise":
            # Its input (the rank-r activations) is replicated, but every rank back-propagates only
            # its own output columns into it: the gradient of that input is a partial sum, and so
            # would be lora_A's weight gradient and the adapter's share of dx. Identity forward,
            # all-reduce of the input gradient in backward, as for the base layer.
            _wrap_forward(module, "colwise", tp_group)
            continue
        if leaf == "lora_A" and kind == "rowwise":
            _wrap_forward(module, "rowwise", tp_group)
            continue
        if sp_state is not None:
            _wrap_forward_sp(module, kind, sp_state)
        else:
            _wrap_forward(module, kind, tp_group)
    # Per-head norm weights see only this rank's heads: their gradients are partial sums. Under
    # sequence parallelism every replicated parameter inside the blocks sees only this rank's
    # tokens; the embedding does not (the gradient of the token shard is gathered before it).
    for name, p in model.named_parameters():
        if name.endswith(("q_norm.weight", "k_norm.weight")):
            p._tp_partial_grad = True
        elif sp_state is not None and not getattr(p, "_tp_sharded", False) \
                and "embed" not in name:
            p._tp_partial_grad = True
    model._sp = sp_state
    model._tp_group = tp_group
    return model


def unshard(local: torch.Tensor, meta, group) -> torch.Tensor:
    """Full tensor from this rank's shard (a collective over ``group``). ``meta`` is the
    ``_tp_meta`` tag ``apply_tp`` leaves on a sharded parameter: ``("rows", sections)`` for
    column-parallel layers (each section of output features was split separately, so that a fused
    q/k/v or gate/up weight keeps whole heads per rank) or ``("cols", [in_features])``."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    kind, sections = meta
    if kind == "cols":
        return torch.cat(parts, dim=1)
    out, start = [], 0
    for n in sections:
        per = n // world
        out.extend(p[start:start + per] for p in parts)
        start += per
    return torch.cat(out, dim=0)


def reshard(full: torch.Tensor, meta, rank: int, world: int) -> torch.Tensor:
    """Inverse of ``unshard``: this rank's shard of a full tensor."""
    kind, sections = meta
    if kind == "cols":
        per = full.shape[1] // world
        return full[:, rank * per:(rank + 1) * per].contiguous()
    return _shard_rows(full, sections, rank, world)


def tp_sharded(p: nn.Parameter) -> bool:
    return bool(getattr(p, "_tp_sharded", False))
