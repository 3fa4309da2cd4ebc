"""Pipeline-parallel helpers: split points and per-stage module names.

As in the reference (lset/distributed/pp.py:4-33) these are planning helpers only: nothing
schedules pipeline stages, ``pp_size`` stays 1 in every supported configuration, and the 3-D mesh
``("pp", "dp", "tp")`` exists for forward compatibility.
"""
from __future__ import annotations

from typing import Dict, List


def get_pp_split_points(num_layers: int, pp_size: int) -> Dict[str, str]:
    """``{"layers.k": "BEGINNING"}`` for the first layer of every stage but the first."""
    if pp_size <= 1:
        return {}
    per = num_layers // pp_size
    extra = num_layers % pp_size
    points, start = {}, 0
    for stage in range(pp_size - 1):
        start += per + (1 if stage < extra else 0)
        points[f"layers.{start}"] = "BEGINNING"
    return points


def get_stage_module_names(num_layers: int, pp_size: int, has_embeddings_name: str = "embed_tokens",
                           final_norm_name: str = "norm") -> List[List[str]]:
    """Module names per stage: embeddings on the first stage, the final norm on the last."""
    per = num_layers // max(1, pp_size)
    extra = num_layers % max(1, pp_size)
    stages, start = [], 0
    for stage in range(max(1, pp_size)):
        n = per + (1 if stage < extra else 0)
        names = [f"layers.{i}" for i in range(start, start + n)]
        if stage == 0:
            names.insert(0, has_embeddings_name)
        if stage == pp_size - 1 or pp_size <= 1:
            names.append(final_norm_name)
        stages.append(names)
        start += n
    return stages
