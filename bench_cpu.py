"""CPU configuration of the comparison: BERT-base-style encoder embedder, fp32, one process.

    python bench_cpu.py [--steps 20] [--impl ours|reference|both]

12 layers, hidden 768, 12 heads, FFN 3072 GELU, post-LayerNorm, learned positions (512), vocab
30522, N(0, 0.02) init; mean pooling over the attention mask + L2 normalisation; InfoNCE with
in-batch negatives at temperature 0.05; 8 (query, positive) pairs per step, token ids U[1000, 30521],
query lengths U[8, 32], passage lengths U[32, 128], right-padded; AdamW lr 2e-5.

``ours`` runs ``lset_b200.train.engine.TrainingEngine`` on the CPU (the eager fp32 path that also
serves as the numerics oracle of the GPU kernels); ``reference`` runs the unmodified reference from
``baseline/_ref`` — its model class, ``BiEncoderTask`` and ``torch.optim.AdamW``, which is what its
engine does at world size 1 — on the same batches. One JSON line per implementation: seconds per
step (wall clock, after 2 untimed steps), pairs/s, first and last loss.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

CFG = dict(vocab_size=30522, hidden_size=768, intermediate_size=3072, num_hidden_layers=12,
           num_attention_heads=12, max_position_embeddings=512, type_vocab_size=2,
           layer_norm_eps=1e-12, hidden_act="gelu", pad_token_id=0)
PAIRS, TEMP, LR, WARM = 8, 0.05, 2e-5, 2


def make_samples(n_steps, seed=1234):
    gen = torch.Generator().manual_seed(seed)

    def seq(lo, hi):
        n = int(torch.randint(lo, hi + 1, (1,), generator=gen))
        return {"input_ids": torch.randint(1000, 30522, (n,), generator=gen).tolist(),
                "attention_mask": [1] * n}

    return [{"query": seq(8, 32), "positive": seq(32, 128)} for _ in range(n_steps * PAIRS)]


def line(impl, steps, secs, losses, extra=None):
    out = {"impl": impl, "metric": "pairs/sec, BERT-base embedder, CPU fp32, 8 pairs/step",
           "value": PAIRS / secs, "unit": "pairs/s", "s_per_step": secs, "steps": steps,
           "warmup": WARM, "first_loss": losses[0], "last_loss": losses[-1], "dtype": "fp32",
           "data": "synthetic", "threads": torch.get_num_threads()}
    out.update(extra or {})
    print(json.dumps(out), flush=True)


def run_ours(steps, samples):
    from lset_b200.models import BertConfig
    from lset_b200.train.data.collator import RightPadCollator
    from lset_b200.train.engine import TrainingEngine

    coll = RightPadCollator(0)
    eng = TrainingEngine("bert", None, dataset=None, batch_size=PAIRS, lr=LR, max_steps=10**9,
                         grad_clip=0.0, temperature=TEMP, packed=False, log_interval=0,
                         scheduler_type="constant", model_config=BertConfig(**CFG), collator=coll,
                         device="cpu", pooling="mean", weight_decay=0.01)
    batches = [coll(samples[i * PAIRS:(i + 1) * PAIRS]) for i in range(steps + WARM)]
    losses = []
    for i, b in enumerate(batches):
        if i == WARM:
            t0 = time.perf_counter()
        losses.append(float(eng.train_step(b)))
    secs = (time.perf_counter() - t0) / steps
    line("ours", steps, secs, losses[WARM:])


def run_reference(steps, samples):
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "lset")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/lset is not installed"}))
        return
    for k in [k for k in sys.modules if k == "lset" or k.startswith("lset.")]:
        del sys.modules[k]
    sys.path.insert(0, ref_root)
    try:
        from lset.models import get_model_spec
        from lset.tasks.bi_encoder import BiEncoderTask
        from lset.train.data.collator import RightPadCollator
    except Exception as exc:  # pragma: no cover - depends on the machine
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {exc!r}"[:300]}))
        return
    spec = get_model_spec("bert")
    torch.manual_seed(42)
    cfg = spec.config_cls(**{k: v for k, v in CFG.items()
                             if k in spec.config_cls.__dataclass_fields__})
    model = spec.model_cls(cfg)
    for p in model.parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, 0.0, 0.02)
    task = BiEncoderTask(pooling="mean", temperature=TEMP)
    opt = torch.optim.AdamW(model.parameters(), lr=LR, weight_decay=0.01)
    coll = RightPadCollator(0)
    batches = [coll(samples[i * PAIRS:(i + 1) * PAIRS]) for i in range(steps + WARM)]
    losses = []
    for i, b in enumerate(batches):
        if i == WARM:
            t0 = time.perf_counter()
        out = task(model, b["query"], b["doc"])
        out["loss"].backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(out["loss"]))
    secs = (time.perf_counter() - t0) / steps
    line("reference", steps, secs, losses[WARM:])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference", "both"], default="both")
    args = ap.parse_args()
    samples = make_samples(args.steps + WARM)
    if args.impl in ("ours", "both"):
        run_ours(args.steps, samples)
    if args.impl in ("reference", "both"):
        run_reference(args.steps, samples)


if __name__ == "__main__":
    main()
