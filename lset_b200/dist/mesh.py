"""Device-mesh construction: ``("dp", "tp")`` for data x tensor parallelism, ``("pp", "dp", "tp")``
when a pipeline dimension is requested (cf. lset/distributed/mesh.py:7-26)."""
from __future__ import annotations

from torch.distributed.device_mesh import init_device_mesh


def build_mesh(dp_size: int = 1, tp_size: int = 1, pp_size: int = 1, device_type: str = "cuda"):
    if pp_size > 1:
        return init_device_mesh(device_type, (pp_size, dp_size, tp_size),
                                mesh_dim_names=("pp", "dp", "tp"))
    return init_device_mesh(device_type, (dp_size, tp_size), mesh_dim_names=("dp", "tp"))
