"""Process-wide switches for the op layer.

The reference toggles its fused kernels through ``LSET_DISABLE_FUSED_*`` environment variables read
inside every kernel wrapper (lset/train/main.py:26-37, lset/kernels/rmsnorm.py:204,
lset/kernels/qk_norm_rope.py:541, lset/kernels/double_residual_rmsnorm.py:282). Here the switches
are an explicit options object that ``configure`` fills from the config; the same environment
variables are still honoured. A disabled switch makes the corresponding op take its eager path.
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass
class RuntimeOptions:
    fused: bool = True
    fused_residual_rmsnorm: bool = True
    fused_pool_normalize: bool = True
    fused_layernorm: bool = True
    fused_rmsnorm: bool = True
    fused_qk_norm_rope: bool = True
    fused_double_rmsnorm: bool = True
    block_runner: bool = True       # whole decoder blocks issued by the native block runner
    tp_block_runner: bool = True    # ... also tensor-parallel blocks on a token-sharded stream
    fused_glu_gemm: bool = False    # gated-MLP activation in the epilogue of the gate/up GEMM (measured slower: off)
    attention_backend: str = "auto"  # auto | native | sdpa


_ENV = {
    "fused_residual_rmsnorm": "LSET_DISABLE_FUSED_RESIDUAL_RMSNORM",
    "fused_pool_normalize": "LSET_DISABLE_FUSED_POOL_NORMALIZE",
    "fused_layernorm": "LSET_DISABLE_FUSED_LAYERNORM",
    "fused_rmsnorm": "LSET_DISABLE_FUSED_RMSNORM",
    "fused_qk_norm_rope": "LSET_DISABLE_FUSED_QK_NORM_ROPE",
    "fused_double_rmsnorm": "LSET_DISABLE_FUSED_DOUBLE_RMSNORM",
    "fused_glu_gemm": "LSET_DISABLE_FUSED_GLU_GEMM",
    "block_runner": "LSET_DISABLE_BLOCK_RUNNER",
    "tp_block_runner": "LSET_DISABLE_TP_BLOCK_RUNNER",
}

options = RuntimeOptions()


def configure(**kwargs) -> RuntimeOptions:
    for k, v in kwargs.items():
        if not hasattr(options, k):
            raise ValueError(f"unknown runtime option {k}")
        setattr(options, k, v)
    if options.attention_backend in ("flash_attn", "varlen_attn"):
        options.attention_backend = "native"  # reference backend names map to the native kernel
    return options


def enabled(name: str) -> bool:
    """True when the native kernel behind ``name`` may be used."""
    if not options.fused:
        return False
    env = _ENV.get(name)
    if env and os.environ.get(env, "0") == "1":
        return False
    return bool(getattr(options, name, True))
