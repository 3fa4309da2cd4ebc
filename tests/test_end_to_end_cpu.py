"""End to end on the CPU from a Hugging Face style checkpoint directory (config.json,
model.safetensors, tokenizer.json) and a JSONL corpus: the training script, ``cli train`` with a
YAML file and overrides, resume from the newest checkpoint, and loading the result for evaluation.
Mirrors the reference's integration tier (tests/test_integration.py, tests/test_cli.py), which needs
local checkpoints; here the checkpoint is a random tiny Qwen3 written by ``transformers``.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

T = pytest.importorskip("transformers")

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORDS = ["alpha", "beta", "gamma", "delta", "query", "passage", "vector", "search", "model", "token",
         "kernel", "tensor", "memory", "gradient", "batch", "index", "what", "is"]


def _model_dir(path):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    vocab = {"[UNK]": 0, **{w: i + 1 for i, w in enumerate(WORDS)},
             **{str(i): len(WORDS) + 1 + i for i in range(64)}}
    tok = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = Whitespace()
    cfg = T.Qwen3Config(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                        max_position_embeddings=256)
    torch.manual_seed(0)
    T.Qwen3Model(cfg).save_pretrained(str(path))
    tok.save(str(path / "tokenizer.json"))
    return path


def _run(args, **kw):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=REPO)
    return subprocess.run([sys.executable, *args], cwd=kw.pop("cwd", REPO), env=env,
                          capture_output=True, text=True, timeout=600)


def test_training_script_from_checkpoint_dir(tmp_path):
    model = _model_dir(tmp_path / "model")
    out = tmp_path / "out"
    r = _run([os.path.join(REPO, "scripts", "train_qwen3_embed.py"), "--model", str(model),
              "--data", str(tmp_path / "train.jsonl"), "--make-data", "24", "--batch-size", "4",
              "--max-steps", "3", "--max-seq-length", "64", "--packed", "--output-dir", str(out)])
    assert r.returncode == 0, r.stderr[-2000:]
    assert "step=" in r.stdout and "loss=" in r.stdout
    rows = [json.loads(line) for line in open(tmp_path / "train.jsonl")]
    assert len(rows) == 24 and {"query", "positive", "negatives"} <= set(rows[0])


def test_cli_train_resume_and_eval_loading(tmp_path):
    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(32):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positive": " ".join(WORDS[(i + j) % 16] for j in range(12)),
                                 "negatives": [" ".join(WORDS[(i + 3 * j) % 16] for j in range(9))]}) + "\n")
    out = tmp_path / "run"
    cfg = tmp_path / "cfg.yaml"
    cfg.write_text(f"""
model:
  path: {model}
data:
  train_path: {data}
  max_seq_length: 48
  num_hard_negatives: 1
training:
  batch_size: 4
  lr: 1.0e-3
  max_steps: 4
  scheduler: constant
  temperature: 0.05
packing:
  enabled: true
checkpoint:
  save_steps: 2
  output_dir: {out}
logging:
  log_interval: 1
""")
    r = _run(["-m", "lset_b200.cli", "train", "--config", str(cfg)])
    assert r.returncode == 0, r.stderr[-2000:]
    steps = sorted(d for d in os.listdir(out) if d.startswith("step_"))
    assert "step_2" in steps and "step_4" in steps
    assert os.path.exists(out / "config.yaml")
    assert os.path.exists(out / "step_4" / "checkpoint.pt") and os.path.exists(out / "step_4" / "meta.pt")

    # resume: two more steps from the newest checkpoint, through a dotted override
    r2 = _run(["-m", "lset_b200.cli", "train", "--config", str(cfg), "--training.max_steps", "6",
               "--checkpoint.resume_from", str(out / "step_4")])
    assert r2.returncode == 0, r2.stderr[-2000:]
    logged = [int(tok.split("=")[1]) for line in r2.stdout.splitlines() if line.startswith("step=")
              for tok in line.split()[:1]]
    assert logged == [4, 5], logged        # the log line carries the index of the step it ran
    assert os.path.exists(out / "step_6" / "meta.pt")

    # the trained weights load back into the model class and differ from the initial checkpoint
    from lset_b200.models import detect_model_type, get_model_spec

    spec = get_model_spec(detect_model_type(str(model)))
    net = spec.model_cls(spec.config_cls.from_hf_json(str(model / "config.json")))
    net.load_state_dict(spec.weight_converter(str(model)))
    before = {k: v.clone() for k, v in net.state_dict().items()}
    blob = torch.load(out / "step_6" / "checkpoint.pt", weights_only=False)
    net.load_state_dict(blob["model"])
    assert blob["step"] == 6
    assert any(not torch.equal(before[k], v) for k, v in net.state_dict().items())

    # and the evaluation wrapper encodes text with the checkpoint's tokenizer
    from lset_b200.eval.mteb_evaluator import LSETMTEBModel

    w = LSETMTEBModel.from_pretrained(str(model), device="cpu")
    emb = w.encode([["what is alpha 1", "beta gamma delta"]])
    assert emb.shape == (2, 32)


def _bert_dir(path):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    vocab = {"[PAD]": 0, "[UNK]": 1, **{w: i + 2 for i, w in enumerate(WORDS)},
             **{str(i): len(WORDS) + 2 + i for i in range(64)}}
    tok = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = Whitespace()
    cfg = T.BertConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=4, max_position_embeddings=128)
    torch.manual_seed(0)
    T.BertModel(cfg).save_pretrained(str(path))
    tok.save(str(path / "tokenizer.json"))
    return path


@pytest.mark.parametrize("variant", ["bert_padded_scored_gradcache", "qwen3_lora_ac_matryoshka"])
def test_cli_train_variants(tmp_path, variant):
    """Other corners of the YAML surface through the real CLI: an encoder with padded batches,
    the scored (soft-label) and multi-positive dataset formats, GradCache; LoRA with activation
    checkpointing and matryoshka dims on the decoder."""
    data = tmp_path / "train.jsonl"
    bert = variant.startswith("bert")
    model = _bert_dir(tmp_path / "model") if bert else _model_dir(tmp_path / "model")
    with open(data, "w") as fh:
        for i in range(24):
            q = f"what is {WORDS[i % 16]} {i}"
            docs = [" ".join(WORDS[(i + k * j) % 16] for j in range(6 + k)) for k in range(1, 4)]
            if bert:
                row = {"query": q, "documents": [{"text": d, "score": float(3 - k)}
                                                 for k, d in enumerate(docs)]}
            else:
                row = {"query": q, "positives": docs[:2], "negatives": docs[2:]}
            fh.write(json.dumps(row) + "\n")
    out = tmp_path / "run"
    extra = ("packing:\n  enabled: false\ngrad_cache:\n  enabled: true\n  chunk_size: 2\n" if bert else
             "packing:\n  enabled: true\nlora:\n  enabled: true\n  r: 4\n  alpha: 8\n"
             "activation_checkpoint:\n  enabled: true\n  mode: selective\n")
    cfg = tmp_path / "cfg.yaml"
    cfg.write_text(f"model:\n  path: {model}\ndata:\n  train_path: {data}\n  max_seq_length: 32\n"
                   f"  num_hard_negatives: 1\ntraining:\n  batch_size: 4\n  lr: 1.0e-3\n  max_steps: 3\n"
                   f"  scheduler: cosine\n  warmup_steps: 1\n  temperature: 0.05\n"
                   + ("" if bert else "  matryoshka_dims: 16,32\n") + extra +
                   f"checkpoint:\n  save_steps: 3\n  output_dir: {out}\nlogging:\n  log_interval: 1\n")
    r = _run(["-m", "lset_b200.cli", "train", "--config", str(cfg)])
    assert r.returncode == 0, (r.stdout[-1000:], r.stderr[-2000:])
    losses = [float(tok.split("=")[1]) for line in r.stdout.splitlines() if line.startswith("step=")
              for tok in line.split() if tok.startswith("loss=")]
    assert len(losses) == 3 and all(v == v and abs(v) < 1e4 for v in losses), losses
    assert os.path.exists(out / "step_3" / "meta.pt")
    if not bert:
        blob = torch.load(out / "step_3" / "checkpoint.pt", weights_only=False)
        assert any("lora_A" in k for k in blob["model"])


def test_cli_multiprocess_dp_and_tp(tmp_path):
    """``cli train`` with a world size above one re-executes itself under torchrun (gloo on a
    machine without GPUs): sharded data parallelism, tensor parallelism, and both with the
    sequence-parallel scheme. The same global batches give the same losses with and without
    tensor parallelism, and the checkpoint is the sharded (DCP) layout with one file per rank."""
    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(48):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positive": " ".join(WORDS[(i + j) % 16] for j in range(12)),
                                 "negatives": [" ".join(WORDS[(i + 3 * j) % 16] for j in range(9))]}) + "\n")
    (tmp_path / "empty.yaml").write_text("{}\n")
    losses = {}
    for tag, extra in (("dp2", ["--distributed.dp_size", "2"]),
                       ("tp2", ["--distributed.tp_size", "2"]),
                       ("dp2tp2", ["--distributed.dp_size", "2", "--distributed.tp_size", "2",
                                   "--distributed.async_tp", "true"])):
        out = tmp_path / tag
        r = _run(["-m", "lset_b200.cli", "train", "--config", str(tmp_path / "empty.yaml"),
                  "--model.path", str(model), "--data.train_path", str(data),
                  "--data.max_seq_length", "48", "--training.batch_size", "4",
                  "--training.max_steps", "3", "--training.lr", "1e-3", "--packing.enabled", "true",
                  "--checkpoint.save_steps", "3", "--checkpoint.output_dir", str(out),
                  "--logging.log_interval", "1", *extra])
        assert r.returncode == 0, (tag, r.stderr[-2000:])
        losses[tag] = [float(tok.split("=")[1]) for line in r.stdout.splitlines()
                       if line.startswith("step=") for tok in line.split() if tok.startswith("loss=")]
        assert len(losses[tag]) == 3, (tag, r.stdout[-500:])
        files = os.listdir(out / "step_3")
        world = 4 if tag == "dp2tp2" else 2
        assert "meta.pt" in files and ".metadata" in files
        assert sum(f.endswith(".distcp") for f in files) == world
    for a, b in zip(losses["dp2"], losses["dp2tp2"]):
        assert abs(a - b) < 1e-3 * max(1.0, abs(a)), (losses["dp2"], losses["dp2tp2"])


@pytest.mark.parametrize("mode", ["raise", "hang"])
def test_elastic_restart_resumes_from_newest_checkpoint(tmp_path, mode):
    """A rank that fails on the host between steps (injected before step 3 on rank 1, first attempt
    only: an exception, or a host-side hang that the step watchdog ends) takes the worker group
    down; the launcher restarts it (``distributed.max_restarts``) and the job continues from the
    newest complete checkpoint."""
    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(64):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positive": " ".join(WORDS[(i + j) % 16] for j in range(12))}) + "\n")
    (tmp_path / "empty.yaml").write_text("{}\n")
    out = tmp_path / "run"
    env_backup = os.environ.get("LSET_B200_FAIL_AT_STEP")
    os.environ["LSET_B200_FAIL_AT_STEP"] = f"3,1,{mode}"
    try:
        r = _run(["-m", "lset_b200.cli", "train", "--config", str(tmp_path / "empty.yaml"),
                  "--model.path", str(model), "--data.train_path", str(data),
                  "--data.max_seq_length", "48", "--training.batch_size", "4",
                  "--training.max_steps", "5", "--training.lr", "1e-3", "--packing.enabled", "true",
                  "--checkpoint.save_steps", "2", "--checkpoint.output_dir", str(out),
                  "--logging.log_interval", "1", "--distributed.dp_size", "2",
                  "--distributed.max_restarts", "1", "--distributed.step_timeout_s", "15"])
    finally:
        if env_backup is None:
            os.environ.pop("LSET_B200_FAIL_AT_STEP", None)
        else:
            os.environ["LSET_B200_FAIL_AT_STEP"] = env_backup
    assert r.returncode == 0, r.stderr[-3000:]
    assert "[fault injection] rank 1 fails before step 3" in r.stderr
    if mode == "hang":
        assert "[watchdog] rank 1: no training step finished" in r.stderr
    steps = [int(line.split()[0].split("=")[1]) for line in r.stdout.splitlines()
             if line.startswith("step=")]
    # first attempt: steps 0..2, checkpoint after step index 1; second attempt resumes at 2
    assert steps == [0, 1, 2, 2, 3, 4], steps
    assert os.path.exists(out / "step_4" / "meta.pt")
    if mode == "raise":
        # the recovered job logs the losses of a job that never failed
        losses = [float(line.split()[1].split("=")[1]) for line in r.stdout.splitlines()
                  if line.startswith("step=")]
        os.environ.pop("LSET_B200_FAIL_AT_STEP", None)
        clean = _run([a if a != str(out) else str(tmp_path / "clean") for a in r.args[1:]])
        assert clean.returncode == 0, clean.stderr[-2000:]
        ref = [float(line.split()[1].split("=")[1]) for line in clean.stdout.splitlines()
               if line.startswith("step=")]
        assert len(ref) == 5
        assert losses[:3] == pytest.approx(ref[:3], abs=1e-4)
        assert losses[3:] == pytest.approx(ref[2:], abs=1e-4), (losses, ref)


def test_checkpoints_move_between_world_sizes(tmp_path):
    """A sharded (two-rank) checkpoint resumes in a single process and a single-process checkpoint
    resumes on two ranks (``checkpoint.resume_from: auto`` picks the newest complete one)."""
    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(64):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positive": " ".join(WORDS[(i + j) % 16] for j in range(12))}) + "\n")
    (tmp_path / "empty.yaml").write_text("{}\n")

    def run(out, steps, *extra):
        r = _run(["-m", "lset_b200.cli", "train", "--config", str(tmp_path / "empty.yaml"),
                  "--model.path", str(model), "--data.train_path", str(data),
                  "--data.max_seq_length", "48", "--training.batch_size", "4",
                  "--training.max_steps", str(steps), "--training.lr", "1e-3",
                  "--packing.enabled", "true", "--checkpoint.save_steps", "2",
                  "--checkpoint.output_dir", str(out), "--logging.log_interval", "1", *extra])
        assert r.returncode == 0, r.stderr[-2000:]
        return [int(line.split()[0].split("=")[1]) for line in r.stdout.splitlines()
                if line.startswith("step=")]

    two = ("--distributed.dp_size", "2")
    assert run(tmp_path / "a", 2, *two) == [0, 1]
    assert os.path.exists(tmp_path / "a" / "step_2" / ".metadata")
    assert run(tmp_path / "a", 4, "--checkpoint.resume_from", "auto") == [2, 3]
    assert os.path.exists(tmp_path / "a" / "step_4" / "checkpoint.pt")
    assert run(tmp_path / "b", 2) == [0, 1]
    assert run(tmp_path / "b", 4, *two, "--checkpoint.resume_from", "auto") == [2, 3]
    assert os.path.exists(tmp_path / "b" / "step_4" / ".metadata")


def test_tensor_parallel_checkpoints_hold_full_tensors_and_resume_exactly(tmp_path):
    """A tensor-parallel run writes full (unsharded) weights and optimizer moments: resuming it
    under the same layout, under dp2 x tp2 and in a single process continues with the losses of
    the run that was never interrupted."""
    import shutil

    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(64):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positive": " ".join(WORDS[(i + j) % 16] for j in range(12))}) + "\n")
    (tmp_path / "empty.yaml").write_text("{}\n")

    def run(out, steps, *extra):
        r = _run(["-m", "lset_b200.cli", "train", "--config", str(tmp_path / "empty.yaml"),
                  "--model.path", str(model), "--data.train_path", str(data),
                  "--data.max_seq_length", "48", "--training.batch_size", "8",
                  "--training.max_steps", str(steps), "--training.lr", "1e-3",
                  "--training.scheduler", "constant",   # the schedule must not depend on max_steps
                  "--packing.enabled", "true", "--checkpoint.save_steps", "2",
                  "--checkpoint.output_dir", str(out), "--logging.log_interval", "1", *extra])
        assert r.returncode == 0, r.stderr[-2000:]
        return [float(tok.split("=")[1]) for line in r.stdout.splitlines()
                if line.startswith("step=") for tok in line.split() if tok.startswith("loss=")]

    tp2 = ("--distributed.tp_size", "2")
    whole = run(tmp_path / "whole", 4, *tp2)
    assert len(whole) == 4
    first = run(tmp_path / "a", 2, *tp2)
    assert first == pytest.approx(whole[:2], abs=1e-5)
    # the saved tensors have the shapes of the unsharded model
    import torch.distributed.checkpoint as dcp
    meta = dcp.FileSystemReader(str(tmp_path / "a" / "step_2")).read_metadata().state_dict_metadata
    q_shape = tuple(meta["model.layers.0.self_attn.q_proj.weight"].size)
    blob_cfg = json.load(open(model / "config.json"))
    assert q_shape == (blob_cfg["num_attention_heads"] * blob_cfg["head_dim"], blob_cfg["hidden_size"])
    for tag, extra in (("tp2", tp2), ("tp1", ()),
                       ("dp2tp2", ("--distributed.dp_size", "2", "--distributed.tp_size", "2",
                                   "--training.batch_size", "4"))):
        out = tmp_path / f"resume_{tag}"
        shutil.copytree(tmp_path / "a", out)
        rest = run(out, 4, *extra, "--checkpoint.resume_from", "auto")
        assert len(rest) == 2, (tag, rest)
        if tag != "dp2tp2":   # same global batches as the uninterrupted run
            assert rest == pytest.approx(whole[2:], abs=2e-3), (tag, rest, whole)
        else:
            assert all(v == v for v in rest)


@pytest.mark.parametrize("tag,options", [
    ("gradcache_dp2", ["--distributed.dp_size", "2", "--grad_cache.enabled", "true",
                       "--grad_cache.token_budget", "150"]),
    ("lora_tp2", ["--distributed.tp_size", "2", "--lora.enabled", "true", "--lora.r", "4"]),
    ("fp8_tp2", ["--distributed.tp_size", "2", "--fp8.enabled", "true", "--fp8.recipe", "rowwise"]),
    ("padded_sp_dp2_tp2_ac", ["--packing.enabled", "false", "--distributed.dp_size", "2",
                              "--distributed.tp_size", "2", "--distributed.async_tp", "true",
                              "--activation_checkpoint.enabled", "true"]),
])
def test_cli_multiprocess_feature_combinations(tmp_path, tag, options):
    """Feature combinations that involve collectives of their own, through the launcher on CPU:
    GradCache with rank-aligned minibatch plans, LoRA and FP8 layers under tensor parallelism,
    sequence parallelism on padded batches with data parallelism and activation checkpointing."""
    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(64):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positives": [" ".join(WORDS[(i + j) % 16] for j in range(12)),
                                               " ".join(WORDS[(i + 2 * j) % 16] for j in range(7))],
                                 "negatives": [" ".join(WORDS[(i + 3 * j) % 16] for j in range(9))]}) + "\n")
    (tmp_path / "empty.yaml").write_text("{}\n")
    r = _run(["-m", "lset_b200.cli", "train", "--config", str(tmp_path / "empty.yaml"),
              "--model.path", str(model), "--data.train_path", str(data),
              "--data.max_seq_length", "48", "--data.num_hard_negatives", "1",
              "--training.batch_size", "4", "--training.max_steps", "2", "--training.lr", "1e-3",
              "--packing.enabled", "true", "--checkpoint.save_steps", "0",
              "--checkpoint.output_dir", str(tmp_path / "out"), "--logging.log_interval", "1",
              *options])
    assert r.returncode == 0, r.stderr[-2000:]
    losses = [float(tok.split("=")[1]) for line in r.stdout.splitlines() if line.startswith("step=")
              for tok in line.split() if tok.startswith("loss=")]
    assert len(losses) == 2 and all(v == v and abs(v) < 1e4 for v in losses), losses


def test_cli_eval_without_mteb_says_what_is_missing(tmp_path):
    try:
        import mteb  # noqa: F401
        pytest.skip("mteb is installed")
    except ImportError:
        pass
    cfg = tmp_path / "c.yaml"
    cfg.write_text(f"model:\n  path: {tmp_path}\neval:\n  tasks: [STSBenchmark]\n")
    r = _run(["-m", "lset_b200.cli", "eval", "--config", str(cfg)])
    assert r.returncode != 0 and "mteb" in (r.stderr + r.stdout)


def test_run_eval_with_a_stand_in_for_mteb(tmp_path, monkeypatch, capsys):
    """``run_eval`` glue (cf. lset/eval/run.py:10-46) against a stand-in ``mteb`` module: the model
    is loaded from the checkpoint directory, handed to ``mteb.evaluate`` with the configured tasks
    and batch size, and the main score of every task is printed and returned."""
    import types

    model = _model_dir(tmp_path / "model")
    seen = {}

    class Result:
        def __init__(self, name, score):
            self.task_name, self._score = name, score

        def get_score(self):
            return self._score

    def evaluate(wrapper, tasks, encode_kwargs=None):
        seen["tasks"], seen["kwargs"] = list(tasks), encode_kwargs
        emb = wrapper.encode([{"text": ["what is alpha 1", "beta gamma"]}])
        sim = wrapper.similarity(emb, emb)
        return types.SimpleNamespace(task_results=[Result(t, float(sim[0, 1])) for t in tasks])

    fake = types.SimpleNamespace(get_tasks=lambda tasks: list(tasks), evaluate=evaluate)
    monkeypatch.setitem(sys.modules, "mteb", fake)
    from lset_b200.config import LSETConfig
    from lset_b200.eval.run import run_eval

    cfg = LSETConfig()
    cfg.apply_overrides([("model.path", str(model)), ("eval.tasks", "STSBenchmark,SICK-R"),
                         ("eval.batch_size", "16"), ("eval.max_length", "32")])
    scores = run_eval(cfg)
    assert seen["tasks"] == ["STSBenchmark", "SICK-R"] and seen["kwargs"] == {"batch_size": 16}
    assert set(scores) == {"STSBenchmark", "SICK-R"} and all(-1.0 <= v <= 1.0 for v in scores.values())
    out = capsys.readouterr().out
    assert "STSBenchmark: main_score=" in out and "SICK-R: main_score=" in out


def test_parameter_sharded_mode_checkpoints_resume_and_interchange(tmp_path):
    """A run in the parameter-sharded mode saves full tensors like the resident mode: continued in
    the resident mode from its checkpoint it logs the losses of the uninterrupted sharded run."""
    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(64):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positives": [" ".join(WORDS[(i + j) % 16] for j in range(12))],
                                 "negatives": [" ".join(WORDS[(i + 3 * j) % 16] for j in range(9))]}) + "\n")
    (tmp_path / "empty.yaml").write_text("{}\n")

    def run(out, steps, sharded, *extra):
        r = _run(["-m", "lset_b200.cli", "train", "--config", str(tmp_path / "empty.yaml"),
                  "--model.path", str(model), "--data.train_path", str(data),
                  "--data.max_seq_length", "48", "--data.num_hard_negatives", "1",
                  "--training.batch_size", "4", "--training.max_steps", str(steps),
                  "--training.lr", "1e-3", "--training.scheduler", "constant",
                  "--packing.enabled", "true", "--checkpoint.save_steps", "2",
                  "--checkpoint.output_dir", str(out), "--logging.log_interval", "1",
                  "--distributed.dp_size", "2", "--distributed.reshard_after_forward", sharded,
                  *extra])
        assert r.returncode == 0, r.stderr[-2000:]
        return [float(tok.split("=")[1]) for line in r.stdout.splitlines()
                if line.startswith("step=") for tok in line.split() if tok.startswith("loss=")]

    whole = run(tmp_path / "whole", 4, "true")
    assert len(whole) == 4
    assert run(tmp_path / "split", 2, "true") == pytest.approx(whole[:2], abs=1e-4)
    crossed = run(tmp_path / "split", 4, "false", "--checkpoint.resume_from", "auto")
    assert crossed == pytest.approx(whole[2:], abs=1e-3), (crossed, whole)


@pytest.mark.parametrize("layout", [[], ["--distributed.dp_size", "2"]], ids=["single", "dp2"])
def test_checkpoints_do_not_depend_on_fused_projections(tmp_path, layout):
    """A model with fused QKV / gate-up weights writes them under the unfused (reference) names,
    moments included: a run that starts unfused and resumes fused, or the other way round, logs
    the losses of the uninterrupted run, in the single-file and the distributed format."""
    model = _model_dir(tmp_path / "model")
    data = tmp_path / "train.jsonl"
    with open(data, "w") as fh:
        for i in range(64):
            fh.write(json.dumps({"query": f"what is {WORDS[i % 16]} {i}",
                                 "positives": [" ".join(WORDS[(i + j) % 16] for j in range(12))],
                                 "negatives": [" ".join(WORDS[(i + 3 * j) % 16] for j in range(9))]}) + "\n")
    (tmp_path / "empty.yaml").write_text("{}\n")

    def run(out, steps, fused, *extra):
        r = _run(["-m", "lset_b200.cli", "train", "--config", str(tmp_path / "empty.yaml"),
                  "--model.path", str(model), "--data.train_path", str(data),
                  "--data.max_seq_length", "48", "--data.num_hard_negatives", "1",
                  "--training.batch_size", "4", "--training.max_steps", str(steps),
                  "--training.lr", "1e-3", "--training.scheduler", "constant",
                  "--packing.enabled", "true", "--checkpoint.save_steps", "2",
                  "--checkpoint.output_dir", str(out), "--logging.log_interval", "1",
                  "--model.fused_projections", fused, *layout, *extra])
        assert r.returncode == 0, r.stderr[-2000:]
        return [float(tok.split("=")[1]) for line in r.stdout.splitlines()
                if line.startswith("step=") for tok in line.split() if tok.startswith("loss=")]

    whole = run(tmp_path / "whole", 4, "true")
    assert len(whole) == 4
    assert run(tmp_path / "a", 2, "false") == pytest.approx(whole[:2], abs=1e-4)
    rest = run(tmp_path / "a", 4, "true", "--checkpoint.resume_from", "auto")
    assert rest == pytest.approx(whole[2:], abs=1e-3), (rest, whole)
    if layout:       # the distributed format: one direction is enough
        return
    assert run(tmp_path / "b", 2, "true") == pytest.approx(whole[:2], abs=1e-4)
    rest = run(tmp_path / "b", 4, "false", "--checkpoint.resume_from", "auto")
    assert rest == pytest.approx(whole[2:], abs=1e-3), (rest, whole)
    if not layout:
        blob = torch.load(tmp_path / "b" / "step_2" / "checkpoint.pt", map_location="cpu",
                          weights_only=False)
        keys = set(blob["model"])
        assert "layers.0.self_attn.q_proj.weight" in keys and "layers.0.mlp.up_proj.weight" in keys
        assert not any("qkv_proj" in k or "gate_up_proj" in k for k in keys)
