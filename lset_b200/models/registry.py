"""Model registry: name -> ``ModelSpec``; detection of the family from a ``config.json``.

Mirrors the reference's registry surface (lset/models/registry.py:7-79): ``register_model``,
``register_alias``, ``get_model_spec``, ``detect_model_type``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Optional


@dataclass
class ModelSpec:
    config_cls: type
    model_cls: type
    weight_converter: Callable
    tp_plan_fn: Optional[Callable] = None
    default_pooling: str = "last_token"
    default_padding_side: str = "left"
    post_pooling_fn: Optional[Callable] = None
    template: Optional[object] = None


_SPECS: Dict[str, ModelSpec] = {}
_ALIASES: Dict[str, str] = {}

# Hugging Face ``model_type`` -> registry name
_HF_TYPES = {
    "qwen3": "qwen3", "llama": "llama", "llama_bidirec": "llama", "bert": "bert",
    "xlm-roberta": "xlm-roberta", "roberta": "xlm-roberta", "gemma3_text": "embeddinggemma",
}
# fallback: substring of an ``architectures`` entry (lower-cased) -> registry name
_ARCH_HINTS = (("qwen3", "qwen3"), ("llama", "llama"), ("xlmroberta", "xlm-roberta"),
               ("roberta", "xlm-roberta"), ("bert", "bert"), ("gemma", "embeddinggemma"))


def register_model(name: str, spec: ModelSpec) -> None:
    _SPECS[name] = spec


def register_alias(alias: str, name: str) -> None:
    _ALIASES[alias] = name


def get_model_spec(name: str) -> ModelSpec:
    key = _ALIASES.get(name, name)
    if key not in _SPECS:
        known = sorted(set(_SPECS) | set(_ALIASES))
        raise KeyError(f"Unknown model type '{name}'. Registered: {known}")
    return _SPECS[key]


def list_models():
    return sorted(_SPECS)


def detect_model_type(model_path) -> str:
    """Family name for the checkpoint directory (or ``config.json`` path) ``model_path``."""
    p = Path(model_path)
    cfg = p if p.is_file() else p / "config.json"
    if not cfg.exists():
        raise FileNotFoundError(f"config.json not found under {model_path}")
    with open(cfg) as fh:
        raw = json.load(fh)
    mt = raw.get("model_type", "")
    if mt in _HF_TYPES:
        return _HF_TYPES[mt]
    for arch in raw.get("architectures", []) or []:
        low = arch.lower()
        for hint, name in _ARCH_HINTS:
            if hint in low:
                return name
    raise ValueError(f"Cannot determine the model family of {model_path} (model_type={mt!r})")
