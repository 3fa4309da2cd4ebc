"""Checkpoint loading: Hugging Face weight files -> this package's state-dict keys.

Each family is described by a small rule table (prefixes to strip, key prefixes to drop, ordered
substring rewrites); one generic routine applies it, then optionally fuses Q/K/V and gate/up
matrices row-wise for ``fused_projections``. Same resulting keys as the reference's converters
(lset/models/decoder/qwen3/weights.py:10-69, lset/models/encoder/bert/weights.py:37-125,
lset/models/decoder/gemma/weights.py:1-36).
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Sequence, Tuple

import torch


@dataclass(frozen=True)
class KeyRules:
    strip_prefixes: Sequence[str] = ()
    drop_prefixes: Sequence[str] = ()
    rewrites: Sequence[Tuple[str, str]] = ()


DECODER_RULES = KeyRules(strip_prefixes=("model.",), drop_prefixes=("lm_head.",))

_ENCODER_REWRITES = (
    (".gamma", ".weight"), (".beta", ".bias"),
    ("encoder.layer.", "layers."),
    ("attention.self.", "attention."),
    ("attention.output.dense", "attention.dense"),
    ("attention.output.LayerNorm", "attention.LayerNorm"),
    ("intermediate.dense", "mlp.dense_in"),
    ("output.dense", "mlp.dense_out"),
    ("output.LayerNorm", "mlp.LayerNorm"),
)
BERT_RULES = KeyRules(strip_prefixes=("bert.",), drop_prefixes=("pooler.", "cls."),
                      rewrites=_ENCODER_REWRITES)
XLMR_RULES = KeyRules(strip_prefixes=("roberta.",),
                      drop_prefixes=("pooler.", "classifier.", "lm_head."),
                      rewrites=_ENCODER_REWRITES)

# (fused key suffix, source key suffixes) — fused by concatenating rows in this order
_DECODER_FUSIONS = (
    ("self_attn.qkv_proj", ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj")),
    ("mlp.gate_up_proj", ("mlp.gate_proj", "mlp.up_proj")),
)
_ENCODER_FUSIONS = (("attention.qkv_proj", ("attention.query", "attention.key", "attention.value")),)


def read_weight_files(model_dir) -> Dict[str, torch.Tensor]:
    """Merge every ``*.safetensors`` (else ``pytorch_model*.bin``) file of a model directory."""
    model_dir = Path(model_dir)
    merged: Dict[str, torch.Tensor] = {}
    st_files = sorted(model_dir.glob("*.safetensors"))
    if st_files:
        from safetensors.torch import load_file

        for f in st_files:
            merged.update(load_file(str(f)))
        return merged
    bin_files = sorted(model_dir.glob("pytorch_model*.bin"))
    for f in bin_files:
        merged.update(torch.load(str(f), map_location="cpu", weights_only=True))
    if not merged:
        raise FileNotFoundError(f"No model files found in {model_dir}")
    return merged


def apply_rules(state: Dict[str, torch.Tensor], rules: KeyRules) -> Dict[str, torch.Tensor]:
    out = {}
    for key, value in state.items():
        for p in rules.strip_prefixes:
            if key.startswith(p):
                key = key[len(p):]
        if any(key.startswith(p) for p in rules.drop_prefixes):
            continue
        for old, new in rules.rewrites:
            key = key.replace(old, new)
        out[key] = value
    return out


def fuse_projections(state: Dict[str, torch.Tensor], fusions) -> Dict[str, torch.Tensor]:
    """Row-concatenate the listed projections (weights, and biases when all are present)."""
    out = dict(state)
    for fused_suffix, sources in fusions:
        first = sources[0]
        for kind in ("weight", "bias"):
            tail = f"{first}.{kind}"
            for key in [k for k in state if k.endswith(tail)]:
                stem = key[: -len(tail)]
                parts = [f"{stem}{s}.{kind}" for s in sources]
                if all(p in state for p in parts):
                    out[f"{stem}{fused_suffix}.{kind}"] = torch.cat([state[p] for p in parts], dim=0)
                    for p in parts:
                        out.pop(p, None)
    return out


def split_projections(state: Dict[str, torch.Tensor], fusions, sizes_fn) -> Dict[str, torch.Tensor]:
    """Inverse of ``fuse_projections``: ``sizes_fn(fused_key, tensor)`` returns the row counts."""
    out = dict(state)
    for fused_suffix, sources in fusions:
        for kind in ("weight", "bias"):
            tail = f"{fused_suffix}.{kind}"
            for key in [k for k in state if k.endswith(tail)]:
                stem = key[: -len(tail)]
                chunks = torch.split(state[key], sizes_fn(key, state[key]), dim=0)
                for s, c in zip(sources, chunks):
                    out[f"{stem}{s}.{kind}"] = c.clone()
                out.pop(key, None)
    return out


def load_decoder_weights(model_dir, fused_projections: bool = False) -> Dict[str, torch.Tensor]:
    """Qwen3 / Llama / Gemma checkpoints (``model.`` prefix stripped, ``lm_head`` dropped)."""
    state = apply_rules(read_weight_files(model_dir), DECODER_RULES)
    return fuse_projections(state, _DECODER_FUSIONS) if fused_projections else state


load_qwen3_weights = load_decoder_weights
load_llama_weights = load_decoder_weights
load_gemma_weights = load_decoder_weights


def load_bert_weights(model_dir, fused_projections: bool = False) -> Dict[str, torch.Tensor]:
    state = apply_rules(read_weight_files(model_dir), BERT_RULES)
    return fuse_projections(state, _ENCODER_FUSIONS) if fused_projections else state


def load_xlm_roberta_weights(model_dir, fused_projections: bool = False) -> Dict[str, torch.Tensor]:
    state = apply_rules(read_weight_files(model_dir), XLMR_RULES)
    return fuse_projections(state, _ENCODER_FUSIONS) if fused_projections else state


def load_gemma_projection(model_dir):
    """EmbeddingGemma's two post-pooling dense layers (``2_Dense``, ``3_Dense``) when present.
    Returns a list of weight matrices applied in order (``y = x @ Wᵀ``), possibly empty."""
    from safetensors.torch import load_file

    mats = []
    for sub in ("2_Dense", "3_Dense"):
        f = Path(model_dir) / sub / "model.safetensors"
        if f.exists():
            sd = load_file(str(f))
            w = sd.get("linear.weight")
            if w is not None:
                mats.append(w)
    return mats
