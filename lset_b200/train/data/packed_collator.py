"""Packed collators under the reference's module path (lset/train/data/packed_collator.py)."""
from .collator import FixedBudgetPackedCollator, PackedCollator  # noqa: F401
from .packing import _pack_fixed_budget, pack_fixed_budget  # noqa: F401
