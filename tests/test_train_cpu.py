"""Training infrastructure on CPU: scheduler, checkpoint round trip + resume, GradCache
equivalence, gradient accumulation, LoRA, activation checkpointing, watchdog, CLI, PP helpers."""
import math
import os
import subprocess
import sys
import time

import pytest
import torch

from lset_b200.models import Qwen3Config, Qwen3Decoder
from lset_b200.train.data.collator import LeftPadCollator, PackedCollator
from lset_b200.train.data.dataset import SyntheticPairDataset
from lset_b200.train.engine import TrainingEngine
from lset_b200.train.scheduler import build_scheduler, lr_factor

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    return Qwen3Config(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=8)


def _engine(**kw):
    torch.manual_seed(0)
    base = dict(batch_size=4, lr=1e-2, packed=True, model_config=_cfg(), log_interval=0,
                device="cpu", scheduler_type="constant")
    base.update(kw)
    return TrainingEngine("qwen3", None, base.pop("dataset", None), **base)


def _batch(lo, hi, packed=True):
    ds = SyntheticPairDataset(32, 300, (3, 6), (5, 12), seed=5)
    coll = PackedCollator() if packed else LeftPadCollator(0)
    return coll([ds[i] for i in range(lo, hi)])


def test_scheduler_curves():
    assert lr_factor(0, "cosine", 10, 100) == 0.0 and lr_factor(5, "linear", 10, 100) == 0.5
    assert lr_factor(10, "cosine", 10, 110) == 1.0
    assert math.isclose(lr_factor(60, "cosine", 10, 110), 0.5, abs_tol=1e-9)
    assert lr_factor(110, "linear", 10, 110) == 0.0 and lr_factor(500, "cosine", 0, 100) < 1e-9
    assert lr_factor(50, "constant", 0, 100) == 1.0
    assert lr_factor(69, "wsd", 0, 100) == 1.0 and 0 < lr_factor(85, "wsd", 0, 100) < 1.0
    with pytest.raises(ValueError):
        lr_factor(0, "nope", 0, 10)
    eng = _engine(lr=1.0)
    sch = build_scheduler(eng.optimizer, "linear", 2, 12)
    lrs = []
    for _ in range(4):
        lrs.append(sch.get_last_lr()[0])
        sch.step()
    assert lrs == [0.0, 0.5, 1.0, 0.9]
    sd = sch.state_dict()
    sch2 = build_scheduler(eng.optimizer, "linear", 2, 12)
    sch2.load_state_dict(sd)
    assert sch2.get_last_lr() == sch.get_last_lr()


def test_training_reduces_loss_and_checkpoint_roundtrip(tmp_path):
    eng = _engine(output_dir=str(tmp_path))
    first = float(eng.train_step(_batch(0, 4)))
    for _ in range(6):
        last = float(eng.train_step(_batch(0, 4)))
    assert last < first
    ckpt = eng.save(7)
    assert os.path.exists(os.path.join(ckpt, "checkpoint.pt")) and os.path.exists(os.path.join(ckpt, "meta.pt"))
    blob = torch.load(os.path.join(ckpt, "checkpoint.pt"), weights_only=False)
    assert set(blob) == {"model", "optimizer", "step"} and blob["step"] == 7
    assert "layers.0.self_attn.q_proj.weight" in blob["model"]
    st0 = blob["optimizer"]["state"][0]
    assert set(st0) == {"step", "exp_avg", "exp_avg_sq"} and blob["optimizer"]["param_groups"][0]["lr"] == 1e-2
    nxt = float(eng.train_step(_batch(4, 8)))

    from lset_b200.train.checkpoint import latest_checkpoint, load_checkpoint

    assert latest_checkpoint(str(tmp_path)) == ckpt
    eng2 = _engine(output_dir=str(tmp_path))
    assert load_checkpoint(eng2.model, eng2.optimizer, ckpt, store=eng2.store) == 7
    assert abs(float(eng2.train_step(_batch(4, 8))) - nxt) < 1e-5


def test_torch_adamw_equivalence():
    eng = _engine(grad_clip=0.0, weight_decay=0.01)
    ref = Qwen3Decoder(_cfg())
    ref.load_state_dict({k: v.clone() for k, v in eng.model.state_dict().items()})
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    from lset_b200.tasks.bi_encoder import BiEncoderTask

    task = BiEncoderTask()
    for s in range(3):
        b = _batch(4 * s, 4 * s + 4)
        eng.train_step(b)
        opt.zero_grad()
        task(ref, b["query"], b["doc"])["loss"].backward()
        opt.step()
    for (n, p), (_, q) in zip(eng.model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p, q, atol=2e-5), n


@pytest.mark.parametrize("packed", [True, False])
def test_grad_cache_equals_standard(packed):
    outs = []
    for gc in (False, True):
        eng = _engine(packed=packed, use_grad_cache=gc, gc_chunk_size=3,
                      gc_token_budget=30 if packed else None)
        loss = eng.forward_backward(_batch(0, 8, packed), True)
        outs.append((float(loss), torch.cat([g.flat_grad for g in eng.store.groups]).clone()))
    assert abs(outs[0][0] - outs[1][0]) < 1e-5
    assert (outs[0][1] - outs[1][1]).abs().max() < 1e-4


def test_gradient_accumulation_matches_big_batch_direction():
    eng = _engine(gradient_accumulation_steps=2, grad_clip=0.0)
    eng.train_step(_batch(0, 4))
    assert eng.optimizer.step_count == 0
    eng.train_step(_batch(4, 8))
    assert eng.optimizer.step_count == 1 and eng.micro_step == 2


def test_planner_and_policies():
    from lset_b200.train.grad_cache import MinibatchBackward, plan_minibatches, slice_feature
    from lset_b200.train.grad_cache.planner import token_budget_plan

    assert token_budget_plan([5, 5, 5, 20, 1], 10) == [(0, 2), (2, 3), (3, 4), (4, 5)]
    b = _batch(0, 5)["doc"]
    assert plan_minibatches(b, 2) == [(0, 2), (2, 4), (4, 5)]
    sub = slice_feature(b, 1, 3)
    assert sub["cu_seqlens"][0] == 0 and sub["position_ids"][0] == 0
    pad = _batch(0, 4, packed=False)["query"]
    s2 = slice_feature(pad, 0, 1)
    assert s2["attention_mask"].all()  # padding columns trimmed

    class FakeDS:
        module = None

        def __init__(self):
            self.calls = []

        def set_gradient_accumulation_boundary(self, b):
            self.calls.append(("boundary", b))

        def backward(self, t):
            self.calls.append(("backward",))

    class FakeFSDP:
        def __init__(self):
            self.calls = []

        def set_requires_gradient_sync(self, f):
            self.calls.append(f)

        def set_reshard_after_backward(self, f):
            pass

    ds = FakeDS()
    rt = MinibatchBackward.for_model(ds, is_ga_boundary=True)
    rt.backward(torch.zeros(()), False)
    rt.backward(torch.zeros(()), True)
    assert ds.calls == [("boundary", False), ("backward",), ("boundary", True), ("backward",)]
    fs = FakeFSDP()
    rt = MinibatchBackward.for_model(fs, is_ga_boundary=False)
    t = torch.zeros((), requires_grad=True)
    rt.backward(t * 1, True)
    assert fs.calls == [False]
    plans, real = MinibatchBackward.for_model(torch.nn.Linear(1, 1)).align_minibatches([[(0, 1)], [(0, 2), (2, 3)]])
    assert real == [1, 2] and plans[1] == [(0, 2), (2, 3)]


def test_rand_context_reproduces_dropout():
    from lset_b200.train.grad_cache import RandContext

    x = torch.ones(100)
    ctx = RandContext(x)
    a = torch.nn.functional.dropout(x, 0.5)
    with ctx:
        b = torch.nn.functional.dropout(x, 0.5)
    assert torch.equal(a, b)


def test_lora_training_only_touches_adapters(tmp_path):
    eng = _engine(lora=True, lora_r=4, lora_alpha=8.0)
    names = [n for n, p in eng.model.named_parameters() if p.requires_grad]
    assert names and all("lora_" in n for n in names)
    base = eng.model.layers[0].self_attn.q_proj.base_linear.weight.clone()
    for _ in range(2):
        eng.train_step(_batch(0, 4))
    assert torch.equal(base, eng.model.layers[0].self_attn.q_proj.base_linear.weight)
    assert eng.model.layers[0].self_attn.q_proj.lora_B.weight.abs().sum() > 0
    from lset_b200.train.lora import load_lora_weights, save_lora_weights

    f = str(tmp_path / "adapter.pt")
    save_lora_weights(eng.model, f)
    eng2 = _engine(lora=True, lora_r=4, lora_alpha=8.0)
    load_lora_weights(eng2.model, f)
    assert torch.equal(eng2.model.layers[1].mlp.down_proj.lora_A.weight,
                       eng.model.layers[1].mlp.down_proj.lora_A.weight)


@pytest.mark.parametrize("mode", ["full", "selective"])
def test_activation_checkpointing_same_grads(mode):
    a = _engine()
    b = _engine(activation_checkpoint=True, ac_mode=mode, ac_ratio=1.0)
    la, lb = a.forward_backward(_batch(0, 4), True), b.forward_backward(_batch(0, 4), True)
    assert torch.allclose(la, lb, atol=1e-6)
    for ga, gb in zip(a.store.groups, b.store.groups):
        assert torch.allclose(ga.flat_grad, gb.flat_grad, atol=1e-5)
    assert list(a.model.state_dict()) == list(b.model.state_dict())


def test_watchdog_fires_and_beats():
    from lset_b200.train.watchdog import StepWatchdog

    hits = []
    w = StepWatchdog(0.2, on_timeout=hits.append, poll_s=0.05, exit_process=False)
    w.start()
    for _ in range(6):
        time.sleep(0.05)
        w.beat()
    assert not w.fired
    time.sleep(0.5)
    w.stop()
    assert w.fired and hits and hits[0] > 0.2


def test_pp_helpers():
    from lset_b200.dist.pp import get_pp_split_points, get_stage_module_names

    assert get_pp_split_points(28, 1) == {}
    assert get_pp_split_points(8, 2) == {"layers.4": "BEGINNING"}
    stages = get_stage_module_names(5, 2)
    assert stages[0][0] == "embed_tokens" and stages[-1][-1] == "norm"
    assert sum(len([n for n in s if n.startswith("layers.")]) for s in stages) == 5


def test_cli_routing(tmp_path):
    def run(*args):
        return subprocess.run([sys.executable, "-m", "lset_b200.cli", *args], cwd=REPO,
                              capture_output=True, text=True)

    r = run()
    assert r.returncode == 1 and "Commands:" in r.stdout
    assert run("help").returncode == 0
    r = run("bogus")
    assert r.returncode == 1 and "Unknown command" in r.stdout
    r = run("train")
    assert r.returncode == 1 and "--config is required" in r.stdout
    cfg = tmp_path / "c.yaml"
    cfg.write_text("cuda_graph:\n  enabled: true\ncompile:\n  enabled: true\n")
    r = run("train", "--config", str(cfg))
    assert r.returncode != 0 and "redundant" in (r.stderr + r.stdout)


def test_cuda_graph_validation():
    from lset_b200.train.cuda_graph import validate_cuda_graph_config

    validate_cuda_graph_config(False, False, False)
    validate_cuda_graph_config(True, False, False, token_budget=4096)
    for args in ((True, False, False), (False, True, False), (False, False, True)):
        with pytest.raises(ValueError):
            validate_cuda_graph_config(*args)


def test_chunked_encoder_weighted_merge():
    from lset_b200.eval.chunked_encoder import chunk_ids, encode_chunked, plan_streams

    assert chunk_ids(list(range(10)), 4, 1) == [[0, 1, 2, 3], [3, 4, 5, 6], [6, 7, 8, 9]]
    assert sorted(sum(plan_streams([5, 9, 3, 2], 10), [])) == [0, 1, 2, 3]
    from lset_b200.models import BertConfig, BertEncoder
    from lset_b200.models.layers import init_normal_

    torch.manual_seed(0)
    m = BertEncoder(BertConfig(vocab_size=50, hidden_size=16, intermediate_size=32,
                               num_hidden_layers=1, num_attention_heads=2, max_position_embeddings=32))
    init_normal_(m, 0.1)
    tok = lambda texts: [[(ord(c) % 40) + 5 for c in t] for t in texts]  # noqa: E731
    out = encode_chunked(m, tok, None, ["abcdefghij", "xy"], device="cpu", chunk_len=4, overlap=0,
                         token_budget=8)
    assert out.shape == (2, 16) and abs(float((out[0] ** 2).sum()) - 1.0) < 1e-5
    with pytest.raises(ValueError):
        encode_chunked(m, tok, None, ["abcdefghij"], device="cpu", pooling="cls", chunk_len=4)


def test_main_grad_is_found_through_detached_aliases():
    """Checkpointed blocks hand the backward detached aliases of the parameters: the fp32
    accumulator is still found (by storage address), and an entry dies with its parameter."""
    import gc

    from lset_b200.ops._grads import main_grad_of, register_main_grad

    p = torch.nn.Parameter(torch.zeros(4, 4))
    p.main_grad = torch.ones(4, 4)
    register_main_grad(p)
    alias = p.detach()
    assert main_grad_of(p) is p.main_grad and main_grad_of(alias) is p.main_grad
    assert main_grad_of(p.detach()[:2]) is None          # a different shape is not the parameter
    del p, alias
    gc.collect()
    fresh = [torch.zeros(4, 4) for _ in range(8)]        # may reuse the freed address
    assert all(main_grad_of(t) is None for t in fresh)


def test_cpu_embedding_scatters_into_accumulators():
    """The CPU lookup matches aten's embedding (values and gradients); with an fp32 accumulator
    registered the rows are added into it and no dense gradient is returned."""
    import torch.nn.functional as F

    from lset_b200.ops import _grads
    from lset_b200.ops.embedding import embedding

    torch.manual_seed(0)
    tab = torch.randn(50, 16, requires_grad=True)
    pos = torch.randn(12, 16, requires_grad=True)
    ids = torch.randint(0, 50, (3, 7))
    pid = torch.arange(7)[None, :]
    out = embedding(ids, tab, 2.0, extra=[(pid, pos)])
    ref = (F.embedding(ids, tab) + F.embedding(pid.expand_as(ids), pos)) * 2.0
    assert torch.allclose(out, ref)
    g = torch.randn_like(out)
    gt, gp = torch.autograd.grad(out, [tab, pos], g)
    rt, rp = torch.autograd.grad(ref, [tab, pos], g)
    assert torch.allclose(gt, rt, atol=1e-6) and torch.allclose(gp, rp, atol=1e-6)

    tab2 = tab.detach().clone().requires_grad_()
    tab2.main_grad = torch.ones(50, 16)
    _grads.register_main_grad(tab2)
    out2 = embedding(ids, tab2, 2.0)
    out2.backward(g)
    assert tab2.grad is None
    r2, = torch.autograd.grad(F.embedding(ids, tab) * 2.0, [tab], g)
    assert torch.allclose(tab2.main_grad, r2 + 1.0, atol=1e-6)
