"""Parity with Hugging Face ``transformers`` on randomly initialised tiny models (CPU, fp32).

Each family is built in ``transformers`` from a small config, saved with ``save_pretrained`` and
loaded back through this package's own path — model-type detection, config parsing, weight-name
conversion, model class — and the last hidden states are compared. This is the check the reference
runs against local checkpoints (tests/models/test_qwen3_hf_match.py:6,63 and its siblings for BERT,
BGE-M3, Llama-nemotron and EmbeddingGemma, ``atol=1e-4``); random weights need no downloads.
"""
import pytest
import torch

T = pytest.importorskip("transformers")

from lset_b200.models import detect_model_type, get_model_spec  # noqa: E402


def _load_ours(path, fused=False):
    name = detect_model_type(path)
    spec = get_model_spec(name)
    cfg = spec.config_cls.from_hf_json(f"{path}/config.json")
    model = spec.model_cls(cfg, fused_projections=True) if fused else spec.model_cls(cfg)
    sd = spec.weight_converter(path, fused_projections=True) if fused else spec.weight_converter(path)
    model.load_state_dict(sd, strict=True)
    return name, model.eval()


def _hf(cls, cfg, tmp_path):
    torch.manual_seed(0)
    hf = cls(cfg).eval()
    for p in hf.parameters():          # non-trivial norm weights and biases too
        torch.nn.init.normal_(p, 0.0, 0.05)
    hf.save_pretrained(str(tmp_path))
    return hf


def _ids():
    torch.manual_seed(1)
    ids = torch.randint(3, 90, (2, 9))
    mask = torch.ones(2, 9, dtype=torch.long)
    mask[1, 6:] = 0                    # right padding on the second row
    return ids, mask


def _close(a, b, mask=None, atol=1e-4):
    if mask is not None:
        a, b = a * mask[..., None], b * mask[..., None]
    err = float((a - b).abs().max())
    assert err < atol, err


@pytest.mark.parametrize("fused", [False, True])
def test_qwen3(tmp_path, fused):
    cfg = T.Qwen3Config(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                        max_position_embeddings=64)
    hf = _hf(T.Qwen3Model, cfg, tmp_path)
    name, ours = _load_ours(str(tmp_path), fused)
    assert name == "qwen3"
    ids, _ = _ids()
    with torch.no_grad():
        _close(hf(input_ids=ids).last_hidden_state, ours(ids)["hidden_states"])


def test_llama_bidirectional(tmp_path):
    cfg = T.LlamaConfig(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    hf = _hf(T.LlamaModel, cfg, tmp_path)
    name, ours = _load_ours(str(tmp_path))
    assert name == "llama"
    ids, _ = _ids()
    everything = torch.zeros(2, 1, 9, 9)          # additive 4-D mask: no position is hidden
    with torch.no_grad():
        got = ours(ids)["hidden_states"]
        _close(hf(input_ids=ids, attention_mask=everything).last_hidden_state, got)
        # and it is not the causal model
        assert float((hf(input_ids=ids).last_hidden_state - got).abs().max()) > 1e-3


def test_bert_with_padding(tmp_path):
    cfg = T.BertConfig(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                       num_attention_heads=4, max_position_embeddings=32)
    hf = _hf(T.BertModel, cfg, tmp_path)
    name, ours = _load_ours(str(tmp_path))
    assert name == "bert"
    ids, mask = _ids()
    with torch.no_grad():
        _close(hf(input_ids=ids, attention_mask=mask).last_hidden_state,
               ours(ids, attention_mask=mask)["hidden_states"], mask, atol=1e-5)


def test_xlm_roberta_position_offset(tmp_path):
    cfg = T.XLMRobertaConfig(vocab_size=100, hidden_size=64, intermediate_size=128,
                             num_hidden_layers=2, num_attention_heads=4,
                             max_position_embeddings=40, pad_token_id=1)
    hf = _hf(T.XLMRobertaModel, cfg, tmp_path)
    name, ours = _load_ours(str(tmp_path))
    assert name == "xlm-roberta"
    ids, mask = _ids()
    with torch.no_grad():
        _close(hf(input_ids=ids, attention_mask=mask).last_hidden_state,
               ours(ids, attention_mask=mask)["hidden_states"], mask, atol=1e-5)


def test_embedding_gemma_backbone(tmp_path):
    cfg = T.Gemma3TextConfig(vocab_size=100, hidden_size=64, intermediate_size=128,
                             num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                             head_dim=16, max_position_embeddings=64, sliding_window=32,
                             query_pre_attn_scalar=16)
    hf = _hf(T.Gemma3TextModel, cfg, tmp_path)
    name, ours = _load_ours(str(tmp_path))
    assert name == "embeddinggemma"
    ids, _ = _ids()                                # 9 tokens: inside the sliding window
    with torch.no_grad():
        _close(hf(input_ids=ids).last_hidden_state, ours(ids)["hidden_states"])
