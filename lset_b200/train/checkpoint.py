"""Checkpoint save / load.

Layout and schemas of the reference (lset/train/checkpoint.py:9-53): ``output_dir/step_{N}/``
holds ``checkpoint.pt = {"model", "optimizer", "step"}`` for a single process, or a
``torch.distributed.checkpoint`` (DCP) directory with the keys ``model`` and ``optimizer`` when a
process group is up; rank 0 writes ``meta.pt = {"step": N}`` last, so a directory is complete iff
``meta.pt`` exists. Model keys are the module's FQNs, optimizer state follows torch's AdamW
schema. On top of that, ``extra.pt`` (scheduler, RNG and sampler position) makes resumption exact;
readers that do not know it can ignore it.

With the sharded runtime the model entry holds the fp32 master weights (what the reference keeps
in its FSDP2 parameters); frozen parameters and buffers are stored as they are.

Fused projections (``model.fused_projections``: one ``qkv_proj`` / ``gate_up_proj`` weight) are
written under the reference's names, split into ``q_proj`` / ``k_proj`` / ``v_proj`` (``query`` /
``key`` / ``value`` for BERT) and ``gate_proj`` / ``up_proj``, weights, biases and both AdamW moments,
and fused again on the way in: a checkpoint does not depend on the flag, and the reference, which
has no fused modules, can read it.
"""
from __future__ import annotations

import os
import re
from pathlib import Path
from typing import Optional

import torch
import torch.distributed as dist


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def _tp_of(store):
    """``(group, rank, world)`` of the tensor-parallel group the store was built with."""
    group = getattr(store, "tp_group", None) if store is not None else None
    if group is None or not _dist_on() or dist.get_world_size(group) == 1:
        return None, 0, 1
    return group, dist.get_rank(group), dist.get_world_size(group)


def _tp_metas(model) -> dict:
    """``name -> _tp_meta`` for every tensor-parallel-sharded parameter (in module order, the same
    on every rank, so the gathers below pair up)."""
    return {n: p._tp_meta for n, p in model.named_parameters() if hasattr(p, "_tp_meta")}


# ---------------------------------------------------------------------- fused projections
def _fusions(model) -> list:
    """``[(fused module FQN, [(part module FQN, share), ...])]`` for every fused projection that is
    a plain linear layer (an adapter wrapped around a fused projection has no unfused twin and
    keeps its names). Shares are the parts' relative numbers of output rows."""
    from torch import nn

    out = []
    for mname, m in model.named_modules():
        pre = mname + "." if mname else ""
        if getattr(m, "fused_qkv", False) and isinstance(getattr(m, "qkv_proj", None), nn.Linear):
            if hasattr(m, "num_kv_heads"):
                parts = [("q_proj", m.num_heads), ("k_proj", m.num_kv_heads), ("v_proj", m.num_kv_heads)]
            else:
                parts = [("query", 1), ("key", 1), ("value", 1)]
            out.append((pre + "qkv_proj", [(pre + n, w) for n, w in parts]))
        if getattr(m, "fused_gate_up", False) and isinstance(getattr(m, "gate_up_proj", None), nn.Linear):
            out.append((pre + "gate_up_proj", [(pre + "gate_proj", 1), (pre + "up_proj", 1)]))
    return out


def _split_rows(t: torch.Tensor, shares) -> list:
    total = sum(shares)
    rows = [t.shape[0] * w // total for w in shares]
    assert sum(rows) == t.shape[0], (t.shape, shares)
    return list(torch.split(t, rows, dim=0))


def _unfuse_state(sd: dict, fusions) -> dict:
    for fused, parts in fusions:
        for suffix in ("weight", "bias"):
            t = sd.pop(f"{fused}.{suffix}", None)
            if t is not None:
                for (name, _), piece in zip(parts, _split_rows(t, [w for _, w in parts])):
                    sd[f"{name}.{suffix}"] = piece.contiguous()
    return sd


def _fuse_state(sd: dict, fusions) -> dict:
    for fused, parts in fusions:
        for suffix in ("weight", "bias"):
            keys = [f"{name}.{suffix}" for name, _ in parts]
            if f"{fused}.{suffix}" not in sd and all(k in sd for k in keys):
                sd[f"{fused}.{suffix}"] = torch.cat([sd.pop(k) for k in keys], dim=0)
    return sd


def _optim_layout(model, fusions) -> Optional[list]:
    """The model's trainable parameters in optimizer order as ``("plain", index)`` or
    ``("fused", {suffix: index}, parts)`` entries (the weight and bias of one fused projection form
    one entry); None when nothing is fused."""
    by_prefix = {fused: parts for fused, parts in fusions}
    if not by_prefix:
        return None
    layout, seen, idx = [], {}, 0
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        prefix, _, suffix = name.rpartition(".")
        if prefix in by_prefix and suffix in ("weight", "bias"):
            if prefix not in seen:
                seen[prefix] = ("fused", {}, by_prefix[prefix])
                layout.append(seen[prefix])
            seen[prefix][1][suffix] = idx
        else:
            layout.append(("plain", idx))
        idx += 1
    return layout


def _entry(state: dict, idx):
    return state.get(idx, state.get(str(idx)))


def _unfuse_optim(osd: dict, layout) -> dict:
    """Optimizer state renumbered for the unfused module order: per part its weight, then its
    bias, the moments split by rows."""
    state, out = osd["state"], {}
    for item in layout:
        if item[0] == "plain":
            ent = _entry(state, item[1])
            if ent is not None:
                out[len(out)] = ent
            else:
                out[len(out)] = None
            continue
        _, idxs, parts = item
        shares = [w for _, w in parts]
        pieces = {}
        for suffix, i in idxs.items():
            ent = _entry(state, i)
            pieces[suffix] = None if ent is None else {
                "step": ent["step"],
                "exp_avg": _split_rows(ent["exp_avg"], shares),
                "exp_avg_sq": _split_rows(ent["exp_avg_sq"], shares)}
        for j in range(len(parts)):
            for suffix in ("weight", "bias"):
                if suffix not in idxs:
                    continue
                e = pieces[suffix]
                out[len(out)] = None if e is None else {
                    "step": e["step"].clone() if torch.is_tensor(e["step"]) else e["step"],
                    "exp_avg": e["exp_avg"][j].contiguous(),
                    "exp_avg_sq": e["exp_avg_sq"][j].contiguous()}
    n = len(out)
    groups = [dict(g, params=list(range(n))) for g in (osd.get("param_groups") or [])][:1]
    return {"state": {k: v for k, v in out.items() if v is not None}, "param_groups": groups}


def _fuse_optim(osd: dict, layout) -> dict:
    """Inverse of ``_unfuse_optim`` for a state dict written in the unfused numbering."""
    state, out, src = osd["state"], {}, 0
    own = sum(1 if it[0] == "plain" else len(it[1]) for it in layout)
    for item in layout:
        if item[0] == "plain":
            ent = _entry(state, src)
            if ent is not None:
                out[item[1]] = ent
            src += 1
            continue
        _, idxs, parts = item
        got = {suffix: [] for suffix in idxs}
        for _ in parts:
            for suffix in ("weight", "bias"):
                if suffix in idxs:
                    got[suffix].append(_entry(state, src))
                    src += 1
        for suffix, i in idxs.items():
            ents = got[suffix]
            if all(e is not None for e in ents):
                out[i] = {"step": ents[0]["step"],
                          "exp_avg": torch.cat([e["exp_avg"] for e in ents], dim=0),
                          "exp_avg_sq": torch.cat([e["exp_avg_sq"] for e in ents], dim=0)}
    groups = [dict(g, params=list(range(own))) for g in (osd.get("param_groups") or [])][:1]
    return {"state": out, "param_groups": groups}


def _optim_entries(osd: dict) -> int:
    groups = osd.get("param_groups") or []
    if groups and "params" in groups[0]:
        return sum(len(g["params"]) for g in groups)
    return len(osd["state"])


def model_state(model, store=None) -> dict:
    """Full (unsharded) model tensors by FQN. Data-parallel shards are gathered by the store;
    tensor-parallel shards are re-assembled over the tensor-parallel group, so a checkpoint holds
    the same tensors whatever the parallel layout that wrote it."""
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    if store is not None:
        for name, t in store.named_master_tensors():
            sd[name] = t.detach()
    group, _, tpw = _tp_of(store)
    if tpw > 1:
        from ..dist.tp import unshard

        for name, meta in _tp_metas(model).items():
            sd[name] = unshard(sd[name], meta, group)
    return _unfuse_state(sd, _fusions(model))


def load_model_state(model, sd: dict, store=None, strict: bool = True) -> None:
    sd = _fuse_state(dict(sd), _fusions(model))
    _, tpr, tpw = _tp_of(store)
    if tpw > 1:
        from ..dist.tp import reshard

        for name, meta in _tp_metas(model).items():
            if name in sd:
                sd[name] = reshard(sd[name], meta, tpr, tpw)
    model.load_state_dict({k: v for k, v in sd.items()}, strict=strict)
    if store is not None:
        store.load_master(sd)


def optimizer_state(optimizer, model=None, store=None) -> dict:
    """``optimizer.state_dict()`` with the moments of tensor-parallel shards re-assembled."""
    osd = optimizer.state_dict()
    group, _, tpw = _tp_of(store)
    if tpw > 1 and model is not None:
        from ..dist.tp import unshard

        canon = store.canonical_index()
        for p in sorted(store.trainable_parameters(), key=lambda q: canon[id(q)]):
            meta, idx = getattr(p, "_tp_meta", None), canon[id(p)]
            if meta is not None and idx in osd["state"]:
                ent = osd["state"][idx]
                for k in ("exp_avg", "exp_avg_sq"):
                    ent[k] = unshard(ent[k], meta, group)
    layout = _optim_layout(model, _fusions(model)) if model is not None else None
    return _unfuse_optim(osd, layout) if layout is not None else osd


def load_optimizer_state(optimizer, osd: dict, store=None, model=None) -> None:
    layout = _optim_layout(model, _fusions(model)) if model is not None else None
    if layout is not None:
        own = sum(1 if it[0] == "plain" else len(it[1]) for it in layout)
        if _optim_entries(osd) != own:      # written in the unfused numbering
            osd = _fuse_optim(osd, layout)
    _, tpr, tpw = _tp_of(store)
    if tpw > 1:
        from ..dist.tp import reshard

        state = dict(osd["state"])
        canon = store.canonical_index()
        for p in store.trainable_parameters():
            meta, idx = getattr(p, "_tp_meta", None), canon[id(p)]
            ent = state.get(idx, state.get(str(idx)))
            if meta is not None and ent is not None:
                ent = dict(ent)
                for k in ("exp_avg", "exp_avg_sq"):
                    ent[k] = reshard(ent[k], meta, tpr, tpw)
                state[idx] = ent
                state.pop(str(idx), None)
        osd = {"state": state, "param_groups": osd.get("param_groups")}
    optimizer.load_state_dict(osd)


def save_checkpoint(model, optimizer, step: int, output_dir: str, store=None,
                    extra: Optional[dict] = None) -> str:
    ckpt_dir = os.path.join(output_dir, f"step_{step}")
    os.makedirs(ckpt_dir, exist_ok=True)
    msd = model_state(model, store)                   # collective under sharding
    osd = optimizer_state(optimizer, model, store)    # collective under sharding
    rank0 = (not _dist_on()) or dist.get_rank() == 0
    if _dist_on() and dist.get_world_size() > 1:
        import torch.distributed.checkpoint as dcp

        # every rank holds the full tensors after the gathers above; DCP writes them de-duplicated
        dcp.save({"model": msd, "optimizer": _flatten_optim(osd)}, checkpoint_id=ckpt_dir)
    elif rank0:
        torch.save({"model": {k: v.cpu() for k, v in msd.items()}, "optimizer": _to_cpu(osd),
                    "step": step}, os.path.join(ckpt_dir, "checkpoint.pt"))
    if rank0:
        if extra is not None:
            torch.save(extra, os.path.join(ckpt_dir, "extra.pt"))
        torch.save({"step": step}, os.path.join(ckpt_dir, "meta.pt"))
    if _dist_on():
        dist.barrier()
    return ckpt_dir


def load_checkpoint(model, optimizer, ckpt_dir: str, store=None) -> int:
    """Restore model and optimizer; returns the saved step (0 when ``meta.pt`` is missing)."""
    single = os.path.join(ckpt_dir, "checkpoint.pt")
    if os.path.exists(single):
        blob = torch.load(single, map_location="cpu", weights_only=False)
        load_model_state(model, blob["model"], store)
        load_optimizer_state(optimizer, blob["optimizer"], store, model)
    else:
        import torch.distributed.checkpoint as dcp

        msd = model_state(model, store)
        osd = _flatten_optim(optimizer_state(optimizer, model, store))
        target = {"model": msd, "optimizer": osd}
        dcp.load(target, checkpoint_id=ckpt_dir)
        load_model_state(model, target["model"], store)
        load_optimizer_state(optimizer, _unflatten_optim(target["optimizer"]), store, model)
    meta = os.path.join(ckpt_dir, "meta.pt")
    if os.path.exists(meta):
        return int(torch.load(meta, map_location="cpu", weights_only=False)["step"])
    return 0


def load_extra(ckpt_dir: str) -> Optional[dict]:
    f = os.path.join(ckpt_dir, "extra.pt")
    return torch.load(f, map_location="cpu", weights_only=False) if os.path.exists(f) else None


def latest_checkpoint(output_dir: str) -> Optional[str]:
    """Newest complete ``step_*`` directory under ``output_dir`` (complete = has ``meta.pt``)."""
    best, best_step = None, -1
    root = Path(output_dir)
    if not root.is_dir():
        return None
    for d in root.iterdir():
        m = re.fullmatch(r"step_(\d+)", d.name)
        if m and (d / "meta.pt").exists() and int(m.group(1)) > best_step:
            best, best_step = str(d), int(m.group(1))
    return best


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


def _flatten_optim(osd: dict) -> dict:
    """DCP wants string keys: ``state.{idx}.{field}`` tensors plus the param_groups object."""
    flat = {"param_groups": osd["param_groups"]}
    for idx, ent in osd["state"].items():
        for k, v in ent.items():
            flat[f"state.{idx}.{k}"] = v
    return flat


def _unflatten_optim(flat: dict) -> dict:
    state = {}
    for k, v in flat.items():
        if k.startswith("state."):
            _, idx, field = k.split(".", 2)
            state.setdefault(int(idx), {})[field] = v
    return {"state": state, "param_groups": flat["param_groups"]}
