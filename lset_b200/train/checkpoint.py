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
    return sd


def load_model_state(model, sd: dict, store=None, strict: bool = True) -> None:
    _, tpr, tpw = _tp_of(store)
    if tpw > 1:
        from ..dist.tp import reshard

        sd = dict(sd)
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
    return osd


def load_optimizer_state(optimizer, osd: dict, store=None) -> None:
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
        load_optimizer_state(optimizer, blob["optimizer"], store)
    else:
        import torch.distributed.checkpoint as dcp

        msd = model_state(model, store)
        osd = _flatten_optim(optimizer_state(optimizer, model, store))
        target = {"model": msd, "optimizer": osd}
        dcp.load(target, checkpoint_id=ckpt_dir)
        load_model_state(model, target["model"], store)
        load_optimizer_state(optimizer, _unflatten_optim(target["optimizer"]), store)
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
