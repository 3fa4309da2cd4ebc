"""Pooling entry points under the reference's module names (lset/models/pooling.py,
lset/models/packed_pooling.py); the implementations live in ``lset_b200.ops.pooling``."""
from ..ops.pooling import normalize, packed_pool, pool  # noqa: F401
