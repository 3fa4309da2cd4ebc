"""``train(config)`` across model families, dataset formats and training options on the CPU, from
Hugging Face style checkpoint directories written by ``transformers`` (random tiny models):
every combination must run two optimizer steps with a finite loss. Covers the reference's
multi-model integration tier (tests/test_multi_model_training.py, tests/test_integration.py)
without local checkpoints."""
import json
import math

import pytest
import torch

T = pytest.importorskip("transformers")

from lset_b200.config import LSETConfig  # noqa: E402
from lset_b200.train.main import train  # noqa: E402

WORDS = ["alpha", "beta", "gamma", "delta", "query", "passage", "vector", "search", "model", "token",
         "kernel", "tensor", "memory", "gradient", "batch", "index", "what", "is"]


def _hf_configs():
    dec = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    enc = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=4)
    return {
        "qwen3": (T.Qwen3Model, T.Qwen3Config(head_dim=8, **dec)),
        "llama": (T.LlamaModel, T.LlamaConfig(**dec)),
        "gemma": (T.Gemma3TextModel, T.Gemma3TextConfig(head_dim=8, sliding_window=64,
                                                         query_pre_attn_scalar=8, **dec)),
        "bert": (T.BertModel, T.BertConfig(max_position_embeddings=128, **enc)),
        "xlmr": (T.XLMRobertaModel, T.XLMRobertaConfig(max_position_embeddings=140, pad_token_id=1,
                                                       **enc)),
    }


@pytest.fixture(scope="module")
def workspace(tmp_path_factory):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    root = tmp_path_factory.mktemp("matrix")
    vocab = {"[PAD]": 0, "[UNK]": 1, **{w: i + 2 for i, w in enumerate(WORDS)},
             **{str(i): len(WORDS) + 2 + i for i in range(64)}}
    dirs = {}
    for name, (cls, cfg) in _hf_configs().items():
        d = root / name
        torch.manual_seed(0)
        cls(cfg).save_pretrained(str(d))
        tok = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
        tok.pre_tokenizer = Whitespace()
        tok.save(str(d / "tokenizer.json"))
        dirs[name] = d
    files = {}
    for fmt in ("pair", "triplet", "multi", "scored"):
        f = root / f"{fmt}.jsonl"
        with open(f, "w") as fh:
            for i in range(24):
                q = f"what is {WORDS[i % 16]} {i}"
                docs = [" ".join(WORDS[(i + k * j) % 16] for j in range(6 + k)) for k in range(1, 4)]
                row = {"pair": {"query": q, "positive": docs[0]},
                       "triplet": {"query": q, "positive": docs[0], "negatives": docs[1:]},
                       "multi": {"query": q, "positives": docs[:2], "negatives": docs[2:]},
                       "scored": {"query": q, "documents": [{"text": d, "score": float(3 - k)}
                                                            for k, d in enumerate(docs)]}}[fmt]
                fh.write(json.dumps(row) + "\n")
        files[fmt] = f
    return root, dirs, files


CASES = [
    ("llama", "pair", {"packing.enabled": "true"}),
    ("llama", "triplet", {"packing.enabled": "false", "model.pooling": "mean"}),
    ("xlmr", "multi", {"packing.enabled": "true"}),
    ("xlmr", "scored", {"packing.enabled": "false"}),
    ("gemma", "triplet", {"packing.enabled": "false"}),
    ("gemma", "pair", {"packing.enabled": "true"}),
    ("qwen3", "triplet", {"packing.enabled": "true", "training.gradient_accumulation_steps": "2",
                          "training.max_steps": "4"}),
    ("qwen3", "pair", {"packing.enabled": "true", "fp8.enabled": "true", "fp8.recipe": "tensorwise"}),
    ("qwen3", "multi", {"packing.enabled": "true", "qlora.enabled": "true", "lora.r": "4"}),
    ("qwen3", "triplet", {"packing.enabled": "true", "grad_cache.enabled": "true",
                          "grad_cache.token_budget": "200"}),
    ("qwen3", "scored", {"packing.enabled": "false", "training.learnable_temperature": "true"}),
    ("bert", "pair", {"packing.enabled": "true", "model.fused_projections": "true",
                      "data.length_sorted": "true"}),
    ("qwen3", "pair", {"packing.enabled": "true", "training.top_k": "2"}),
    ("qwen3", "pair", {"packing.enabled": "true", "cuda_graph.enabled": "true",
                       "cuda_graph.token_budget": "256", "attention.backend": "sdpa",
                       "training.scheduler": "wsd", "training.warmup_steps": "1"}),
    ("qwen3", "triplet", {"packing.enabled": "true", "activation_checkpoint.enabled": "true",
                          "activation_checkpoint.mode": "full", "activation_checkpoint.ratio": "0.5"}),
]


@pytest.mark.parametrize("family,fmt,options", CASES,
                         ids=[f"{a}-{b}-{'+'.join(k.split('.')[0] for k in c if k != 'packing.enabled') or 'plain'}"
                              f"-{'packed' if c['packing.enabled'] == 'true' else 'padded'}"
                              for a, b, c in CASES])
def test_train_runs(workspace, capsys, family, fmt, options):
    root, dirs, files = workspace
    cfg = LSETConfig()
    base = {"model.path": str(dirs[family]), "data.train_path": str(files[fmt]),
            "data.max_seq_length": "32", "data.num_hard_negatives": "1", "training.batch_size": "4",
            "training.lr": "1e-3", "training.max_steps": "2", "training.temperature": "0.05",
            "checkpoint.output_dir": str(root / "out" / f"{family}_{fmt}"),
            "checkpoint.save_steps": "0", "logging.log_interval": "1"}
    base.update(options)
    cfg.apply_overrides(list(base.items()))
    cfg.validate()
    train(cfg)
    out = capsys.readouterr().out
    losses = [float(tok.split("=")[1]) for line in out.splitlines() if line.startswith("step=")
              for tok in line.split() if tok.startswith("loss=")]
    assert len(losses) >= 2 and all(math.isfinite(v) for v in losses), (losses, out[-500:])


@pytest.mark.parametrize("packed,learnable", [("true", "false"), ("false", "false"), ("true", "true")])
def test_resume_continues_mid_epoch_with_the_same_batches(workspace, capsys, packed, learnable):
    """An interrupted run that resumes from its checkpoint sees the batches the uninterrupted run
    would have seen (the order of an epoch depends on seed and epoch only; the checkpoint records
    how far into the epoch it was) and therefore logs the same losses, also across an epoch end.
    With a learnable temperature its value and optimizer moments come back too."""
    root, dirs, files = workspace

    def run(out, max_steps, resume=None):
        cfg = LSETConfig()
        over = {"model.path": str(dirs["qwen3"]), "data.train_path": str(files["triplet"]),
                "data.max_seq_length": "32", "data.num_hard_negatives": "1",
                "training.batch_size": "4", "training.lr": "1e-3", "training.scheduler": "constant",
                "training.max_steps": str(max_steps), "training.temperature": "0.05",
                "packing.enabled": packed, "training.learnable_temperature": learnable,
                "checkpoint.output_dir": str(out),
                "checkpoint.save_steps": "4", "logging.log_interval": "1"}
        if resume:
            over["checkpoint.resume_from"] = resume
        cfg.apply_overrides(list(over.items()))
        train(cfg)
        text = capsys.readouterr().out
        return {int(line.split()[0].split("=")[1]): float(line.split()[1].split("=")[1])
                for line in text.splitlines() if line.startswith("step=")}

    # 24 samples / batch 4 = 6 batches per epoch: steps 4..9 cross the epoch boundary
    whole = run(root / f"whole_{packed}_{learnable}", 10)
    assert sorted(whole) == list(range(10))
    first = run(root / f"split_{packed}_{learnable}", 4)
    rest = run(root / f"split_{packed}_{learnable}", 10, resume="auto")
    assert sorted(rest) == list(range(4, 10))
    for step in range(4):
        assert first[step] == pytest.approx(whole[step], abs=1e-5)
    for step in range(4, 10):
        assert rest[step] == pytest.approx(whole[step], abs=1e-4), (step, rest, whole)


@pytest.mark.parametrize("family,pooling", [("qwen3", "last_token"), ("llama", "mean"),
                                            ("gemma", "mean"), ("bert", "cls"), ("xlmr", "cls")])
def test_eval_wrapper_loads_every_family(workspace, family, pooling):
    """``LSETMTEBModel.from_pretrained`` picks the family's default pooling, encodes through the
    packed forward, and a text gets the same embedding alone as inside a batch."""
    import numpy as np

    from lset_b200.eval.mteb_evaluator import LSETMTEBModel

    _, dirs, _ = workspace
    w = LSETMTEBModel.from_pretrained(str(dirs[family]), device="cpu")
    assert w.pooling == pooling
    texts = ["what is alpha 1", "beta gamma delta kernel tensor memory gradient batch index", "vector"]
    emb = w.encode([texts])
    assert emb.shape == (3, 32) and np.allclose(np.linalg.norm(emb, axis=1), 1.0, atol=1e-4)
    assert np.allclose(w.encode([[texts[1]]])[0], emb[1], atol=1e-5)
