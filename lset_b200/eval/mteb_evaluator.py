"""MTEB model wrapper (cf. lset/eval/mteb_evaluator.py:21-247).

``LSETMTEBModel`` implements what MTEB v2's encoder protocol needs: ``encode(inputs, *, task_metadata,
hf_split, hf_subset, prompt_type, **kw)`` over a DataLoader of ``{"text": [...]}`` batches,
``similarity`` / ``similarity_pairwise`` (cosine) and ``mteb_model_meta``. Texts are tokenised,
packed under a token budget and run through the model's packed path (``encode_chunked``), so long
documents are chunk-averaged under mean pooling and nothing is padded.
"""
from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Iterable, List, Optional

import numpy as np
import torch

from ..models import detect_model_type, get_model_spec
from .chunked_encoder import DEFAULT_CHUNK_LEN, DEFAULT_TOKEN_BUDGET, encode_chunked

log = logging.getLogger(__name__)


class LSETMTEBModel:
    def __init__(self, model, tokenizer, pooling: str = "last_token", max_length: int = 512,
                 device=None, query_prefix: str = "", document_prefix: str = "",
                 model_name: str = "lset-b200/model", revision: str = "local",
                 token_budget: int = DEFAULT_TOKEN_BUDGET, chunked: bool = True,
                 chunk_len: int = DEFAULT_CHUNK_LEN, post_pooling=None):
        self.model = model.eval()
        self.tokenizer = tokenizer
        self.pooling = pooling
        self.max_length = max_length
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.query_prefix, self.document_prefix = query_prefix, document_prefix
        self.model_name, self.revision = model_name, revision
        self.token_budget, self.chunked, self.chunk_len = token_budget, chunked, chunk_len
        self.post_pooling = post_pooling

    @classmethod
    def from_pretrained(cls, model_path: str, pooling: str = "auto", max_length: int = 512,
                        device: Optional[str] = None, dtype=None, **kw) -> "LSETMTEBModel":
        from ..tokenization import load_tokenizer

        name = detect_model_type(model_path)
        spec = get_model_spec(name)
        cfg = spec.config_cls.from_hf_json(str(Path(model_path) / "config.json"))
        model = spec.model_cls(cfg)
        model.load_state_dict(spec.weight_converter(model_path), strict=True)
        dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        dtype = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        model = model.to(device=dev, dtype=dtype)
        pool = spec.default_pooling if pooling in (None, "auto") else pooling
        proj = spec.post_pooling_fn(model_path) if spec.post_pooling_fn is not None else None
        if proj is not None:
            proj = proj.to(device=dev, dtype=dtype)
        return cls(model, load_tokenizer(model_path), pool, max_length, dev,
                   model_name=f"lset-b200/{Path(model_path).name}", post_pooling=proj, **kw)

    # ------------------------------------------------------------------ encoding
    def _tokenize_many(self, texts: List[str]) -> List[List[int]]:
        limit = self.max_length if not (self.chunked and self.pooling == "mean") else None
        out = []
        for t in texts:
            ids = self.tokenizer.encode(t).ids
            out.append(ids[:limit] if limit else ids)
        return out

    def encode_texts(self, texts: List[str], prompt: str = "") -> np.ndarray:
        texts = [prompt + t for t in texts] if prompt else list(texts)
        chunk_len = self.chunk_len if (self.chunked and self.pooling == "mean") else 10**9
        return encode_chunked(self.model, self._tokenize_many, None, texts, device=self.device,
                              pad_id=self._pad_id(), pooling=self.pooling, normalize=True,
                              chunk_len=chunk_len, token_budget=self.token_budget,
                              post_pooling=self.post_pooling)

    def encode(self, inputs: Iterable, *, task_metadata=None, hf_split=None, hf_subset=None,
               prompt_type=None, **kwargs) -> np.ndarray:
        prompt = ""
        if prompt_type is not None:
            kind = getattr(prompt_type, "value", str(prompt_type))
            prompt = self.query_prefix if "query" in kind else self.document_prefix
        chunks = []
        for batch in inputs:
            texts = batch["text"] if isinstance(batch, dict) else list(batch)
            chunks.append(self.encode_texts(list(texts), prompt))
        if not chunks:
            return np.zeros((0, 0), dtype=np.float32)
        return np.concatenate(chunks, axis=0)

    # ------------------------------------------------------------------ similarity
    @staticmethod
    def _t(x):
        return torch.as_tensor(np.asarray(x), dtype=torch.float32)

    def similarity(self, embeddings1, embeddings2) -> torch.Tensor:
        a = torch.nn.functional.normalize(self._t(embeddings1), dim=-1)
        b = torch.nn.functional.normalize(self._t(embeddings2), dim=-1)
        return a @ b.t()

    def similarity_pairwise(self, embeddings1, embeddings2) -> torch.Tensor:
        a = torch.nn.functional.normalize(self._t(embeddings1), dim=-1)
        b = torch.nn.functional.normalize(self._t(embeddings2), dim=-1)
        return (a * b).sum(-1)

    @property
    def mteb_model_meta(self):
        try:
            from mteb.models import ModelMeta
        except Exception:  # pragma: no cover - optional dependency
            return None
        try:
            return ModelMeta(name=self.model_name, revision=self.revision, release_date=None,
                             languages=None, loader=None, n_parameters=None, memory_usage_mb=None,
                             max_tokens=self.max_length, embed_dim=None, license=None,
                             open_weights=True, public_training_code=None,
                             public_training_data=None, framework=["PyTorch"], similarity_fn_name="cosine",
                             use_instructions=bool(self.query_prefix), training_datasets=None)
        except Exception as exc:  # pragma: no cover - depends on the mteb version
            log.warning("could not build ModelMeta: %s", exc)
            return None

    def _pad_id(self) -> int:
        cfg = getattr(self.model, "config", None)
        return int(getattr(cfg, "pad_token_id", 0) or 0)
