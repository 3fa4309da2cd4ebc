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


def model_state(model, store=None) -> dict:
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    if store is not None:
        for name, t in store.named_master_tensors():
            sd[name] = t.detach()
    return sd


def load_model_state(model, sd: dict, store=None, strict: bool = True) -> None:
    model.load_state_dict({k: v for k, v in sd.items()}, strict=strict)
    if store is not None:
        store.load_master(sd)


def save_checkpoint(model, optimizer, step: int, output_dir: str, store=None,
                    extra: Optional[dict] = None) -> str:
    ckpt_dir = os.path.join(output_dir, f"step_{step}")
    os.makedirs(ckpt_dir, exist_ok=True)
    msd = model_state(model, store)          # collective under sharding
    osd = optimizer.state_dict()             # collective under sharding
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
        optimizer.load_state_dict(blob["optimizer"])
    else:
        import torch.distributed.checkpoint as dcp

        msd = model_state(model, store)
        osd = _flatten_optim(optimizer.state_dict())
        target = {"model": msd, "optimizer": osd}
        dcp.load(target, checkpoint_id=ckpt_dir)
        load_model_state(model, target["model"], store)
        optimizer.load_state_dict(_unflatten_optim(target["optimizer"]))
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
