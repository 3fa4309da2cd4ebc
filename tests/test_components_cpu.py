"""CPU tests of the smaller components: tokenizer loading and templates, pooling strategies,
NF4 / QLoRA, MXFP8 emulation, the logger, the MTEB wrapper and the embedding gather."""

import numpy as np
import pytest
import torch
import torch.nn as nn

from lset_b200.models import Qwen3Config, Qwen3Decoder
from lset_b200.models.layers import init_normal_


# ---------------------------------------------------------------------------------- tokenizer
def _tiny_tokenizer(tmp_path):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    vocab = {"[UNK]": 0, "hello": 1, "world": 2, "query": 3, "passage": 4, ":": 5, "a": 6, "b": 7}
    tok = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(tmp_path / "tokenizer.json"))
    return tok


def test_tokenizer_loading_and_templates(tmp_path):
    from lset_b200.tokenization import (QWEN3_EMBEDDING_TEMPLATE, TEMPLATES, EmbeddingTemplate,
                                        load_tokenizer)

    with pytest.raises(FileNotFoundError):
        load_tokenizer(tmp_path)
    _tiny_tokenizer(tmp_path)
    tok = load_tokenizer(tmp_path)
    assert tok.encode("hello world zzz").ids == [1, 2, 0]
    t = EmbeddingTemplate("query : ", "passage : ", query_suffix=" a", document_suffix=" b")
    assert tok.encode(t.format_query("hello")).ids == [3, 5, 1, 6]
    assert tok.encode(t.format_document("world")).ids == [4, 5, 2, 7]
    assert QWEN3_EMBEDDING_TEMPLATE.format_query("x").endswith("Query: x")
    assert QWEN3_EMBEDDING_TEMPLATE.format_document("x") == "x"
    assert TEMPLATES["qwen3"] is QWEN3_EMBEDDING_TEMPLATE


# ---------------------------------------------------------------------------------- pooling
def test_padded_and_packed_pooling_strategies_agree():
    from lset_b200.models.pooling import normalize, packed_pool, pool

    torch.manual_seed(0)
    lens, H = [3, 5, 1, 4], 16
    S = max(lens)
    packed = torch.randn(sum(lens), H)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    seqs = [packed[cu[i]:cu[i + 1]] for i in range(len(lens))]
    right = torch.zeros(len(lens), S, H)
    left = torch.zeros(len(lens), S, H)
    mask_r = torch.zeros(len(lens), S, dtype=torch.long)
    mask_l = torch.zeros(len(lens), S, dtype=torch.long)
    for i, s in enumerate(seqs):
        right[i, :len(s)], mask_r[i, :len(s)] = s, 1
        left[i, S - len(s):], mask_l[i, S - len(s):] = s, 1
    want_mean = torch.stack([s.mean(0) for s in seqs])
    want_last = torch.stack([s[-1] for s in seqs])
    want_cls = torch.stack([s[0] for s in seqs])
    assert torch.allclose(pool(right, mask_r, "mean"), normalize(want_mean), atol=1e-5)
    assert torch.allclose(pool(left, mask_l, "last_token"), normalize(want_last), atol=1e-5)
    assert torch.allclose(pool(right, mask_r, "cls"), normalize(want_cls), atol=1e-5)
    for strategy, want in (("mean", want_mean), ("last_token", want_last), ("cls", want_cls)):
        got = packed_pool(packed, cu, strategy)
        assert torch.allclose(got, normalize(want), atol=1e-5), strategy
        assert torch.allclose(got.norm(dim=-1), torch.ones(len(lens)), atol=1e-5)
    # position-weighted mean: later tokens weigh more; still a convex combination of the tokens
    w = pool(right, mask_r, "weighted_mean")
    pos = torch.arange(1, S + 1)[None, :, None] * mask_r[..., None]
    assert torch.allclose(w, normalize((right * pos).sum(1) / pos.sum(1)), atol=1e-5)


# ---------------------------------------------------------------------------------- NF4 / QLoRA
def test_nf4_roundtrip_and_qlora_application():
    from lset_b200.train.lora import apply_qlora, get_lora_params
    from lset_b200.train.quantization.nf4 import NF4Linear, from_nf4, quantize_linear_nf4, to_nf4

    torch.manual_seed(0)
    w = torch.randn(64, 128) * 0.02
    q = to_nf4(w, block_size=64)
    back = from_nf4(q, torch.float32)
    assert back.shape == w.shape
    # 4-bit normal-float codes: error bounded by half the largest code gap times the block maximum
    blocks = w.reshape(-1, 64)
    bound = blocks.abs().amax(1, keepdim=True) * 0.17
    assert bool(((back.reshape(-1, 64) - blocks).abs() <= bound + 1e-6).all())
    assert float((back - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt()) < 0.12

    lin = nn.Linear(128, 64, bias=True)
    qlin = quantize_linear_nf4(lin)
    assert isinstance(qlin, NF4Linear) and not any(p.requires_grad for p in qlin.parameters())
    x = torch.randn(5, 128)
    assert torch.allclose(qlin(x), nn.functional.linear(x, qlin.dequantized_weight().float(), lin.bias),
                          atol=1e-4)

    cfg = Qwen3Config(vocab_size=64, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=32)
    m = Qwen3Decoder(cfg)
    init_normal_(m, 0.05)
    apply_qlora(m, r=4, alpha=8.0, dropout=0.0, target_modules=None, block_size=64)
    train = get_lora_params(m)
    assert train and all("lora_" in n for n, p in m.named_parameters() if p.requires_grad)
    out = m(torch.arange(10).reshape(2, 5))["hidden_states"]
    out.sum().backward()
    assert all(p.grad is not None for p in train)


# ---------------------------------------------------------------------------------- MXFP8
def test_mxfp8_emulation_block_scales():
    from lset_b200.train.quantization.mx import MXLinear, apply_mxfp8_training, fake_quant_mxfp8

    torch.manual_seed(0)
    x = torch.randn(7, 96) * torch.logspace(-3, 2, 96)   # blocks of very different magnitude
    q = fake_quant_mxfp8(x)
    assert q.shape == x.shape
    # every block of 32 is quantised with its own power-of-two scale: relative error per block
    # stays at e4m3 level no matter how small the block is
    for b in range(3):
        xb, qb = x[:, 32 * b:32 * (b + 1)], q[:, 32 * b:32 * (b + 1)]
        assert float((qb - xb).abs().max() / xb.abs().max()) < 0.07
    # values that are exactly representable survive
    exact = torch.tensor([[1.0, -2.0, 0.5, 448.0] + [0.0] * 28])
    assert torch.equal(fake_quant_mxfp8(exact), exact)
    m = nn.Sequential(nn.Linear(64, 32), nn.Linear(30, 8))
    apply_mxfp8_training(m, "mxfp8_cublas_rceil")
    assert isinstance(m[0], MXLinear) and m[0].rceil and type(m[1]) is nn.Linear
    y = m[0](torch.randn(4, 64))
    y.sum().backward()
    assert m[0].weight.grad is not None
    with pytest.raises(ValueError):
        apply_mxfp8_training(m, "mxfp4")


# ---------------------------------------------------------------------------------- logger
def test_logger_line_format_and_throughput(capsys, tmp_path):
    from lset_b200.train.logging import TrainLogger

    log = TrainLogger(use_wandb=False)
    log.log(7, {"loss": 1.23456789, "lr": 2e-5, "tokens": 12})
    line = capsys.readouterr().out.strip().splitlines()[-1]
    assert line.startswith("step=7") and "loss=1.2346" in line and "tokens=12" in line
    log.reset_throughput()
    tp = log.update_throughput(64, 23000)
    assert tp["samples_per_sec"] > 0 and tp.get("tokens_per_sec", 1) > 0
    log.finish()


# ---------------------------------------------------------------------------------- MTEB wrapper
def test_mteb_wrapper_encodes_and_scores(tmp_path):
    from lset_b200.eval.mteb_evaluator import LSETMTEBModel

    tok = _tiny_tokenizer(tmp_path)
    cfg = Qwen3Config(vocab_size=16, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=16)
    torch.manual_seed(0)
    model = Qwen3Decoder(cfg)
    init_normal_(model, 0.1)
    w = LSETMTEBModel(model, tok, pooling="last_token", max_length=4, device="cpu",
                      query_prefix="query : ")
    emb = w.encode([{"text": ["hello world", "world"]}, {"text": ["a b a b a b"]}])
    assert emb.shape == (3, 32) and np.allclose(np.linalg.norm(emb, axis=1), 1.0, atol=1e-4)
    # truncation to max_length: the long text is cut to four tokens
    assert np.allclose(w.encode([["a b a b a b"]]), w.encode([["a b a b"]]), atol=1e-5)

    class Kind:
        value = "query"

    with_prompt = w.encode([["hello"]], prompt_type=Kind())
    assert np.allclose(with_prompt, w.encode([["query : hello"]]), atol=1e-5)
    sim = w.similarity(emb, emb)
    assert sim.shape == (3, 3) and torch.allclose(sim.diag(), torch.ones(3), atol=1e-4)
    assert torch.allclose(w.similarity_pairwise(emb, emb), torch.ones(3), atol=1e-4)
    assert w.encode([]).shape == (0, 0)


# ---------------------------------------------------------------------------------- gather
def test_gather_single_process_is_identity_with_gradient():
    from lset_b200.dist.gather import gather_for_local_rows, gather_with_grad

    x = torch.randn(4, 8, requires_grad=True)
    for fn in (gather_with_grad, gather_for_local_rows):
        y = fn(x)
        assert torch.equal(y, x)
        g, = torch.autograd.grad(y.pow(2).sum(), x)
        assert torch.allclose(g, 2 * x)


# ---------------------------------------------------------------------------------- chunked encoder
def test_chunked_encoder_planning_cache_retry_and_memmap(tmp_path, monkeypatch):
    import lset_b200.eval.chunked_encoder as ce

    # chunks overlap by `overlap` tokens and cover the whole document
    chunks = ce.chunk_ids(list(range(10)), chunk_len=4, overlap=1)
    assert chunks == [[0, 1, 2, 3], [3, 4, 5, 6], [6, 7, 8, 9]]
    assert ce.chunk_ids([1, 2], 4, 1) == [[1, 2]]
    # streams: longest first, never above the budget unless a single chunk is
    lens = [5, 9, 2, 7, 3]
    streams = ce.plan_streams(lens, budget=10)
    assert sorted(i for s in streams for i in s) == list(range(5))
    assert all(sum(lens[i] for i in s) <= 10 for s in streams) and streams[0][0] == 1
    assert ce.plan_streams([50], budget=10) == [[0]]
    # tokenisation cache: the second call does not tokenise
    calls = []

    def tok(texts):
        calls.append(len(texts))
        return [[ord(c) % 50 + 1 for c in t] for t in texts]

    a = ce.cached_tokenize(tok, ["abc", "de"], tmp_path / "cache")
    b = ce.cached_tokenize(tok, ["abc", "de"], tmp_path / "cache")
    assert a == b and calls == [2]
    assert ce.cached_tokenize(tok, ["abc", "xy"], tmp_path / "cache") != a and calls == [2, 2]

    cfg = Qwen3Config(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=16)
    torch.manual_seed(0)
    model = Qwen3Decoder(cfg).eval()
    init_normal_(model, 0.1)
    texts = ["abcdefghij", "xyz", "", "mnopqrstuvwxyzabcd"]
    ref = ce.encode_chunked(model, tok, None, texts, device="cpu", chunk_len=6, overlap=2,
                            token_budget=64)
    assert ref.shape == (4, 32) and np.allclose(np.linalg.norm(ref, axis=1), 1.0, atol=1e-5)
    # a tiny budget (one chunk per stream) gives the same embeddings
    small = ce.encode_chunked(model, tok, None, texts, device="cpu", chunk_len=6, overlap=2,
                              token_budget=1)
    assert np.allclose(ref, small, atol=1e-5)
    # an out-of-memory error on a multi-chunk stream is retried in halves
    real, state = model.forward, {"raised": 0}

    def flaky(ids, **kw):
        if kw["cu_seqlens"].numel() > 2 and state["raised"] < 2:
            state["raised"] += 1
            raise torch.cuda.OutOfMemoryError("simulated")
        return real(ids, **kw)

    monkeypatch.setattr(model, "forward", flaky)
    again = ce.encode_chunked(model, tok, None, texts, device="cpu", chunk_len=6, overlap=2,
                              token_budget=64)
    assert state["raised"] == 2 and np.allclose(ref, again, atol=1e-5)
    monkeypatch.setattr(model, "forward", real)
    with pytest.raises(ValueError):
        ce.encode_chunked(model, tok, None, texts, device="cpu", pooling="last_token", chunk_len=6)
    # large result sets stream into a memmap on disk
    monkeypatch.setattr(ce, "CPU_STREAM_THRESHOLD", 2)
    mm = ce.encode_chunked(model, tok, None, texts, device="cpu", chunk_len=6, overlap=2,
                           out_path=str(tmp_path / "emb.npy"))
    assert isinstance(mm, np.memmap) and np.allclose(np.load(tmp_path / "emb.npy"), ref, atol=1e-5)


# ---------------------------------------------------------------------------------- tracing / options
def test_roofline_arithmetic_and_peak_loading(tmp_path):
    from lset_b200.utils.tracing import FALLBACK_PEAKS, PhaseTimer, load_peaks, nvtx_range, roofline

    missing = load_peaks(str(tmp_path / "nope.json"))
    assert missing["source"] == "fallback" and missing["hbm_gbs"] == FALLBACK_PEAKS["hbm_gbs"]
    f = tmp_path / "peaks.json"
    f.write_text('{"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "clocks": {"sm": 1900}}')
    peaks = load_peaks(str(f))
    assert peaks["source"] == "measured" and peaks["hbm_gbs"] == 6000.0
    assert peaks["bf16_tflops_sustained"] == FALLBACK_PEAKS["bf16_tflops_sustained"]   # absent key
    # 1 ms for 1.5 PFLOP-ms of math at a 1500 TFLOP/s peak = exactly at the compute roof
    r = roofline(1.0, flops=1.5e12, hbm_bytes=1e9, peaks=peaks)
    assert r["bound"] == "compute" and r["fraction_of_roof"] == pytest.approx(1.0)
    assert r["tflops"] == pytest.approx(1500.0) and r["hbm_gbs"] == pytest.approx(1000.0)
    # a copy of 12 GB in 4 ms at 6000 GB/s: memory-bound, half of the roof
    r = roofline(4.0, hbm_bytes=12e9, peaks=peaks)
    assert r["bound"] == "hbm" and r["fraction_of_roof"] == pytest.approx(0.5)
    # bytes that must cross NVLink bind a fused collective
    r = roofline(1.0, flops=1e9, nvlink_bytes=0.385e9, peaks=peaks)
    assert r["bound"] == "nvlink" and r["fraction_of_roof"] == pytest.approx(0.5)
    assert roofline(1.0, flops=1.4e12, peaks=dict(peaks), sustained=True)["fraction_of_roof"] == \
        pytest.approx(1.0)
    # without a GPU the timer and the NVTX range are inert
    t = PhaseTimer()
    with t.phase("x"), nvtx_range("y"):
        pass
    assert t.report() == {}


def test_runtime_options_and_reference_env_switches(monkeypatch):
    from lset_b200.ops import runtime_options as ro

    saved = dict(vars(ro.options))
    try:
        assert ro.enabled("fused_rmsnorm") and not ro.enabled("fused_glu_gemm")
        monkeypatch.setenv("LSET_DISABLE_FUSED_RMSNORM", "1")      # the reference's switch
        assert not ro.enabled("fused_rmsnorm") and ro.enabled("fused_layernorm")
        monkeypatch.delenv("LSET_DISABLE_FUSED_RMSNORM")
        ro.configure(fused_layernorm=False, attention_backend="flash_attn")
        assert not ro.enabled("fused_layernorm") and ro.options.attention_backend == "native"
        ro.configure(fused=False)
        assert not ro.enabled("fused_rmsnorm")
        with pytest.raises(ValueError):
            ro.configure(no_such_switch=True)
    finally:
        for k, v in saved.items():
            setattr(ro.options, k, v)


def test_gemma_post_pooling_projection_is_applied_between_pooling_and_normalisation(tmp_path):
    """``2_Dense`` / ``3_Dense`` next to a checkpoint become the spec's post-pooling module; the
    task and the chunked encoder apply it before the L2 normalisation."""
    from safetensors.torch import save_file

    from lset_b200.eval.chunked_encoder import encode_chunked
    from lset_b200.models import GemmaConfig, get_model_spec
    from lset_b200.tasks.bi_encoder import BiEncoderTask

    torch.manual_seed(0)
    H = 32
    w_up, w_down = torch.randn(48, H) * 0.2, torch.randn(24, 48) * 0.2
    for sub, w in (("2_Dense", w_up), ("3_Dense", w_down)):
        (tmp_path / sub).mkdir()
        save_file({"linear.weight": w}, str(tmp_path / sub / "model.safetensors"))
    spec = get_model_spec("embeddinggemma")
    proj = spec.post_pooling_fn(tmp_path)
    assert proj is not None and proj.out_features == 24
    assert spec.post_pooling_fn(tmp_path / "2_Dense") is None      # no dense layers there
    cfg = GemmaConfig(vocab_size=128, hidden_size=H, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=16,
                      query_pre_attn_scalar=16, layer_types=["full_attention"])
    model = spec.model_cls(cfg).eval()
    ids = torch.randint(1, 128, (3, 10))
    mask = torch.ones(3, 10, dtype=torch.long)
    mask[1, 6:] = 0
    plain = BiEncoderTask(pooling="mean", normalize=False)
    task = BiEncoderTask(pooling="mean", normalize=True)
    task.set_post_pooling(proj)
    assert "post_pooling" not in dict(task.named_modules())
    with torch.no_grad():
        pooled = plain.encode(model, {"input_ids": ids, "attention_mask": mask})
        emb = task.encode(model, {"input_ids": ids, "attention_mask": mask})
    want = torch.nn.functional.normalize(pooled @ w_up.t() @ w_down.t(), dim=-1)
    assert emb.shape == (3, 24) and torch.allclose(emb, want, atol=1e-5)
    texts = ["a", "b"]
    toks = lambda ts: [[5, 6, 7, 8][: 2 + i] for i, _ in enumerate(ts)]
    out = encode_chunked(model, toks, None, texts, device="cpu", pooling="mean", post_pooling=proj)
    assert out.shape == (2, 24) and abs(float((out[0] ** 2).sum()) - 1.0) < 1e-4


def test_block_runner_arena_sizes_form_a_geometric_series():
    """Arena sizes are rounded up to eight sizes per octave: never smaller than asked for, at most
    12.5 % larger, and token counts a few percent apart share a size (so the caching allocator
    sees a handful of distinct sizes over a run instead of one per batch length)."""
    import random

    from lset_b200.ops.block import _arena_size

    rng = random.Random(0)
    for _ in range(20000):
        n = rng.randint(1, 1 << 40)
        r = _arena_size(n)
        assert n <= r <= n * 1.125 + 1
    assert _arena_size(1000) == 1000                      # small requests stay exact
    sizes = {_arena_size(t * 40960) for t in range(20000, 27000, 50)}   # bytes per token x tokens
    assert len(sizes) <= 5, sorted(sizes)
    assert _arena_size(_arena_size(123456789)) == _arena_size(123456789)
