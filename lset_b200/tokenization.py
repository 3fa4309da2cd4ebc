"""Tokenizer loading and prompt templates (cf. lset/tokenization.py:9-37)."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path


def load_tokenizer(model_path):
    """``tokenizers.Tokenizer`` from ``<model_path>/tokenizer.json``."""
    from tokenizers import Tokenizer

    f = Path(model_path) / "tokenizer.json"
    if not f.exists():
        raise FileNotFoundError(f"tokenizer.json not found in {model_path}")
    return Tokenizer.from_file(str(f))


@dataclass
class EmbeddingTemplate:
    """Text wrapped around queries and documents before tokenisation."""

    query_prefix: str
    document_prefix: str
    query_suffix: str = ""
    document_suffix: str = ""

    def format_query(self, text: str) -> str:
        return f"{self.query_prefix}{text}{self.query_suffix}"

    def format_document(self, text: str) -> str:
        return f"{self.document_prefix}{text}{self.document_suffix}"


QWEN3_EMBEDDING_TEMPLATE = EmbeddingTemplate(
    query_prefix=("Instruct: Given a web search query, retrieve relevant passages that answer "
                  "the query\nQuery: "),
    document_prefix="",
)

TEMPLATES = {"qwen3": QWEN3_EMBEDDING_TEMPLATE}
