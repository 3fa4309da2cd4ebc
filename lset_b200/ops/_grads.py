"""Where a weight gradient goes: the fp32 accumulator of the sharding runtime, found even when the
op only holds a detached alias of the parameter.

``ParamStore`` gives every parameter a ``main_grad`` attribute (a view of its group's flat fp32
buffer) and the ops add weight gradients straight into it. Activation checkpointing hands the
backward *detached copies* of what the recomputed forward saved; they share the parameter's storage
but not its Python attributes. The accumulators are therefore also registered by storage address.
"""
from __future__ import annotations

from typing import Optional

import torch

import weakref

_by_address = {}   # (device, address) -> (weak reference to the owning parameter, accumulator)


def register_main_grad(param: torch.Tensor) -> None:
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        _by_address[(param.device, param.data_ptr())] = (weakref.ref(param), mg)


def main_grad_of(w: torch.Tensor) -> Optional[torch.Tensor]:
    mg = getattr(w, "main_grad", None)
    if mg is not None or not _by_address:
        return mg
    key = (w.device, w.data_ptr())
    entry = _by_address.get(key)
    if entry is None:
        return None
    owner = entry[0]()
    # An entry is valid only while its parameter is alive and still sits at that address: then
    # nothing but an alias of it can have the address. Otherwise the block may have been reused.
    if owner is None or owner.data_ptr() != key[1]:
        del _by_address[key]
        return None
    return entry[1] if entry[1].shape == w.shape else None
