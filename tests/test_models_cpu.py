"""Model families on CPU (eager oracle path): shapes, packed == padded, masks, registry, weights."""
import json

import pytest
import torch

from lset_b200.models import (BertConfig, BertEncoder, EmbeddingGemmaModel, GemmaConfig,
                              LlamaBidirectionalModel, LlamaConfig, Qwen3Config, Qwen3Decoder,
                              detect_model_type, get_model_spec)
from lset_b200.models.layers import init_normal_
from lset_b200.models.weights import (DECODER_RULES, BERT_RULES, apply_rules, fuse_projections,
                                      _DECODER_FUSIONS)
from lset_b200.ops.pooling import packed_pool, pool


def _qwen(**kw):
    return Qwen3Config(vocab_size=200, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=8, **kw)


def _models():
    torch.manual_seed(0)
    yield "qwen3", Qwen3Decoder(_qwen()), True
    yield "llama", LlamaBidirectionalModel(LlamaConfig(
        vocab_size=200, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=8)), False
    yield "gemma", EmbeddingGemmaModel(GemmaConfig(
        vocab_size=200, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
        num_attention_heads=2, num_key_value_heads=1, head_dim=16, query_pre_attn_scalar=16,
        layer_types=["sliding_attention", "full_attention"])), True
    yield "bert", BertEncoder(BertConfig(vocab_size=200, hidden_size=32, intermediate_size=64,
                                         num_hidden_layers=2, num_attention_heads=4)), False


@pytest.mark.parametrize("name,model,causal", list(_models()))
def test_packed_equals_padded(name, model, causal):
    init_normal_(model, 0.05)
    ids = torch.randint(1, 200, (3, 12))
    lens = [12, 7, 3]
    left = name == "qwen3"
    mask = torch.zeros(3, 12, dtype=torch.long)
    seqs = []
    for b, L in enumerate(lens):
        if left:
            mask[b, 12 - L:] = 1
            seqs.append(ids[b, 12 - L:].tolist())
        else:
            mask[b, :L] = 1
            seqs.append(ids[b, :L].tolist())
    padded = model(ids, mask)["hidden_states"]
    assert padded.shape == (3, 12, 32) and not padded.isnan().any()
    flat = torch.tensor([t for s in seqs for t in s])
    cu = torch.tensor([0, 12, 19, 22], dtype=torch.int32)
    pos = torch.cat([torch.arange(L) for L in lens])
    if name == "bert":
        packed = model.forward_packed(flat, pos, cu, 12)["hidden_states"]
    else:
        packed = model.forward_packed(flat, pos, cu, 12)["hidden_states"]
    strategy = "last_token" if left else "mean"
    e_pad = pool(padded, mask, strategy)
    e_pack = packed_pool(packed, cu, strategy)
    if name in ("qwen3", "gemma", "llama") and not left:
        # right-padded rows keep their positions, so packed (positions restart) matches exactly
        pass
    assert torch.allclose(e_pad, e_pack, atol=1e-4), (e_pad - e_pack).abs().max()


def test_causal_vs_bidirectional_information_flow():
    torch.manual_seed(1)
    ids = torch.randint(1, 200, (1, 6))
    ids2 = ids.clone()
    ids2[0, -1] = (ids2[0, -1] + 1) % 200
    q = Qwen3Decoder(_qwen())
    init_normal_(q, 0.05)
    a, b = q(ids)["hidden_states"], q(ids2)["hidden_states"]
    assert torch.allclose(a[0, :-1], b[0, :-1], atol=1e-6)  # causal: earlier tokens unaffected
    l = LlamaBidirectionalModel(LlamaConfig(vocab_size=200, hidden_size=32, intermediate_size=64,
                                            num_hidden_layers=2, num_attention_heads=4,
                                            num_key_value_heads=2, head_dim=8))
    init_normal_(l, 0.05)
    a, b = l(ids)["hidden_states"], l(ids2)["hidden_states"]
    assert (a[0, 0] - b[0, 0]).abs().max() > 1e-7  # bidirectional: first token sees the change


def test_padding_does_not_leak():
    torch.manual_seed(2)
    m = BertEncoder(BertConfig(vocab_size=200, hidden_size=32, intermediate_size=64,
                               num_hidden_layers=2, num_attention_heads=4))
    init_normal_(m, 0.05)
    ids = torch.randint(1, 200, (1, 8))
    mask = torch.tensor([[1, 1, 1, 1, 1, 0, 0, 0]])
    a = m(ids, mask)["hidden_states"][0, :5]
    ids[0, 5:] = 7
    b = m(ids, mask)["hidden_states"][0, :5]
    assert torch.allclose(a, b, atol=1e-6)


def test_lm_logits_and_fused_projection_equivalence():
    torch.manual_seed(3)
    cfg = _qwen()
    m = Qwen3Decoder(cfg)
    init_normal_(m, 0.05)
    out = m(torch.randint(0, 200, (2, 5)), return_lm_logits=True)
    assert out["lm_logits"].shape == (2, 5, 200)
    fused = Qwen3Decoder(cfg, fused_projections=True)
    fused.load_state_dict(fuse_projections(m.state_dict(), _DECODER_FUSIONS))
    ids = torch.randint(0, 200, (2, 5))
    assert torch.allclose(m(ids)["hidden_states"], fused(ids)["hidden_states"], atol=1e-5)


def test_registry_and_detection(tmp_path):
    for name, pooling, side in [("qwen3", "last_token", "left"), ("llama", "mean", "right"),
                                ("bert", "cls", "right"), ("bge-m3", "cls", "right"),
                                ("embeddinggemma", "mean", "right"), ("nv-embed", "mean", "right")]:
        spec = get_model_spec(name)
        assert spec.default_pooling == pooling and spec.default_padding_side == side
    with pytest.raises(KeyError):
        get_model_spec("nope")
    for mt, want in [("qwen3", "qwen3"), ("xlm-roberta", "xlm-roberta"), ("gemma3_text", "embeddinggemma")]:
        (tmp_path / "config.json").write_text(json.dumps({"model_type": mt}))
        assert detect_model_type(tmp_path) == want
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["LlamaBidirectionalModel"]}))
    assert detect_model_type(tmp_path) == "llama"
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "xlm-roberta", "pad_token_id": 1}))
    assert BertConfig.from_hf_json(str(tmp_path / "config.json")).position_offset == 2


def test_weight_key_rules():
    sd = {"model.layers.0.self_attn.q_proj.weight": 1, "lm_head.weight": 2, "model.norm.weight": 3}
    assert set(apply_rules(sd, DECODER_RULES)) == {"layers.0.self_attn.q_proj.weight", "norm.weight"}
    hf = {"bert.encoder.layer.0.attention.self.query.weight": 1,
          "bert.encoder.layer.0.attention.output.dense.bias": 2,
          "bert.encoder.layer.0.attention.output.LayerNorm.gamma": 3,
          "bert.encoder.layer.0.intermediate.dense.weight": 4,
          "bert.encoder.layer.0.output.dense.weight": 5,
          "bert.encoder.layer.0.output.LayerNorm.beta": 6,
          "bert.pooler.dense.weight": 7, "cls.predictions.bias": 8,
          "bert.embeddings.word_embeddings.weight": 9}
    got = set(apply_rules(hf, BERT_RULES))
    assert got == {"layers.0.attention.query.weight", "layers.0.attention.dense.bias",
                   "layers.0.attention.LayerNorm.weight", "layers.0.mlp.dense_in.weight",
                   "layers.0.mlp.dense_out.weight", "layers.0.mlp.LayerNorm.bias",
                   "embeddings.word_embeddings.weight"}


@pytest.mark.parametrize("name,model,causal", list(_models()))
def test_fused_projections_match_separate_for_every_family(name, model, causal):
    """Fused QKV / gate-up (QKV for the encoder) with row-concatenated weights gives the same
    hidden states and the same gradients (the fused gradient is the concatenation)."""
    from lset_b200.models.weights import _ENCODER_FUSIONS

    torch.manual_seed(5)
    init_normal_(model, 0.05)
    fusions = _ENCODER_FUSIONS if name == "bert" else _DECODER_FUSIONS
    fused = type(model)(model.config, fused_projections=True)
    fused.load_state_dict(fuse_projections(model.state_dict(), fusions))
    ids = torch.randint(1, 200, (2, 7))
    a, b = model(ids)["hidden_states"], fused(ids)["hidden_states"]
    assert torch.allclose(a, b, atol=1e-5), (name, float((a - b).abs().max()))
    g = torch.randn_like(a)
    a.backward(g)
    b.backward(g)
    sep, fus = dict(model.named_parameters()), dict(fused.named_parameters())
    for fused_suffix, sources in fusions:
        for key in [k for k in fus if k.endswith(fused_suffix + ".weight")]:
            prefix = key[: -len(fused_suffix + ".weight")]
            want = torch.cat([sep[prefix + s + ".weight"].grad for s in sources])
            rel = float((fus[key].grad - want).abs().max() / (want.abs().max() + 1e-12))
            assert rel < 1e-4, (key, rel)
