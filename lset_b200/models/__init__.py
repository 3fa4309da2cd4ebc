"""Model families and their registration (cf. lset/models/__init__.py:13-95)."""
from . import weights as _w
from .bert import BertEncoder
from .configs import BertConfig, GemmaConfig, LlamaConfig, Qwen3Config
from .decoder import EmbeddingGemmaModel, LlamaBidirectionalModel, Qwen3Decoder
from .parallel_plan import bert_tp_plan, decoder_tp_plan
from .projection import PostPoolingDense, gemma_post_pooling
from .registry import (ModelSpec, detect_model_type, get_model_spec, list_models, register_alias,
                       register_model)

register_model("qwen3", ModelSpec(Qwen3Config, Qwen3Decoder, _w.load_qwen3_weights, decoder_tp_plan,
                                  default_pooling="last_token", default_padding_side="left"))
register_alias("qwen3-embedding", "qwen3")
register_model("llama", ModelSpec(LlamaConfig, LlamaBidirectionalModel, _w.load_llama_weights,
                                  decoder_tp_plan, default_pooling="mean",
                                  default_padding_side="right"))
register_alias("llama-nemotron-embed", "llama")
register_alias("nv-embed", "llama")
register_model("bert", ModelSpec(BertConfig, BertEncoder, _w.load_bert_weights, bert_tp_plan,
                                 default_pooling="cls", default_padding_side="right"))
register_model("xlm-roberta", ModelSpec(BertConfig, BertEncoder, _w.load_xlm_roberta_weights,
                                        bert_tp_plan, default_pooling="cls",
                                        default_padding_side="right"))
register_alias("bge-m3", "xlm-roberta")
register_model("embeddinggemma", ModelSpec(GemmaConfig, EmbeddingGemmaModel, _w.load_gemma_weights,
                                           decoder_tp_plan, default_pooling="mean",
                                           default_padding_side="right",
                                           post_pooling_fn=gemma_post_pooling))

__all__ = [
    "BertConfig", "BertEncoder", "EmbeddingGemmaModel", "GemmaConfig", "LlamaBidirectionalModel",
    "LlamaConfig", "ModelSpec", "PostPoolingDense", "Qwen3Config", "Qwen3Decoder", "detect_model_type",
    "get_model_spec", "list_models", "register_alias", "register_model",
]
