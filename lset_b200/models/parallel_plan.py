"""Tensor-parallel plans: which linear layers are column-sharded (output features split, input
replicated or all-gathered) and which are row-sharded (input features split, output reduced).

A plan maps a module-name pattern (``*`` = layer index) to ``"colwise"`` / ``"rowwise"``, plus
``"sequence"`` for norms whose activations stay token-sharded under sequence parallelism. Same
sharding rules as the reference (lset/models/decoder/qwen3/parallel_plan.py:22-98,
lset/models/encoder/bert/parallel_plan.py:1-31), including the LoRA rule: for a column target the
base and ``lora_B`` are column-sharded, for a row target the base and ``lora_A`` are row-sharded.
"""
from __future__ import annotations

from typing import Dict


def decoder_tp_plan(config=None, use_sequence_parallel: bool = False, use_lora: bool = False,
                    fused_projections: bool = False) -> Dict[str, str]:
    col = (["self_attn.qkv_proj", "mlp.gate_up_proj"] if fused_projections else
           ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "mlp.gate_proj", "mlp.up_proj"])
    row = ["self_attn.o_proj", "mlp.down_proj"]
    plan: Dict[str, str] = {}
    for name in col:
        if use_lora:
            plan[f"layers.*.{name}.base_linear"] = "colwise"
            plan[f"layers.*.{name}.lora_B"] = "colwise"
        else:
            plan[f"layers.*.{name}"] = "colwise"
    for name in row:
        if use_lora:
            plan[f"layers.*.{name}.base_linear"] = "rowwise"
            plan[f"layers.*.{name}.lora_A"] = "rowwise"
        else:
            plan[f"layers.*.{name}"] = "rowwise"
    if use_sequence_parallel and not use_lora:
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                  "post_feedforward_layernorm"):
            plan[f"layers.*.{n}"] = "sequence"
        plan["norm"] = "sequence"
    return plan


def bert_tp_plan(config=None, use_sequence_parallel: bool = False, use_lora: bool = False,
                 fused_projections: bool = False) -> Dict[str, str]:
    col = (["attention.qkv_proj"] if fused_projections else
           ["attention.query", "attention.key", "attention.value"]) + ["mlp.dense_in"]
    row = ["attention.dense", "mlp.dense_out"]
    plan = {f"layers.*.{n}": "colwise" for n in col}
    plan.update({f"layers.*.{n}": "rowwise" for n in row})
    return plan


get_tp_plan = decoder_tp_plan
