"""Model configurations, loadable from a Hugging Face ``config.json``.

Field names and defaults follow the reference's configs
(lset/models/decoder/qwen3/config.py:10-21, lset/models/decoder/llama/config.py:8-31,
lset/models/decoder/gemma/config.py:8-33, lset/models/encoder/bert/config.py:8-37).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import List, Optional


class _HFConfig:
    @classmethod
    def from_hf_json(cls, path: str):
        with open(path) as fh:
            raw = json.load(fh)
        return cls.from_dict(raw)

    @classmethod
    def from_dict(cls, raw: dict):
        names = {f.name for f in dataclasses.fields(cls)}
        kwargs = {k: v for k, v in raw.items() if k in names}
        cfg = cls(**kwargs)
        cfg._post_load(raw)
        return cfg

    def _post_load(self, raw: dict) -> None:  # hook for family-specific derivations
        pass

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)


@dataclass
class Qwen3Config(_HFConfig):
    vocab_size: int = 151669
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    tie_word_embeddings: bool = True
    attention_bias: bool = False
    model_type = "qwen3"


@dataclass
class LlamaConfig(_HFConfig):
    vocab_size: int = 128256
    hidden_size: int = 2048
    intermediate_size: int = 8192
    num_hidden_layers: int = 16
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 64
    max_position_embeddings: int = 131072
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500_000.0
    tie_word_embeddings: bool = True
    attention_bias: bool = False
    rope_scaling: Optional[dict] = None
    model_type = "llama"

    def _post_load(self, raw: dict) -> None:
        if "head_dim" not in raw and self.num_attention_heads:
            self.head_dim = self.hidden_size // self.num_attention_heads


@dataclass
class GemmaConfig(_HFConfig):
    vocab_size: int = 262144
    hidden_size: int = 768
    intermediate_size: int = 1152
    num_hidden_layers: int = 24
    num_attention_heads: int = 3
    num_key_value_heads: int = 1
    head_dim: int = 256
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    rope_local_base_freq: float = 10_000.0
    sliding_window: int = 512
    query_pre_attn_scalar: int = 256
    layer_types: List[str] = field(default_factory=list)
    model_type = "embeddinggemma"


@dataclass
class BertConfig(_HFConfig):
    vocab_size: int = 30522
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"
    pad_token_id: int = 0
    position_offset: int = 0  # XLM-RoBERTa: position ids start at pad_token_id + 1
    model_type = "bert"

    def _post_load(self, raw: dict) -> None:
        if raw.get("model_type", "") in ("xlm-roberta", "roberta"):
            self.position_offset = raw.get("pad_token_id", 1) + 1
