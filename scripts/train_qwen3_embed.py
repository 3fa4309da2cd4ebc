"""Train a Qwen3 embedder from the command line without a YAML file; can generate a small
synthetic JSONL corpus first (counterpart of the reference's scripts/train_qwen3_embed.py, with
working imports).

    python scripts/train_qwen3_embed.py --model ~/models/Qwen3-Embedding-0.6B --make-data 512 \
        --batch-size 32 --max-steps 50 --packed
"""
import argparse
import json
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_corpus(path: str, n: int, seed: int = 0) -> None:
    rng = random.Random(seed)
    words = ["alpha", "beta", "gamma", "delta", "query", "passage", "vector", "search", "model",
             "token", "kernel", "tensor", "memory", "gradient", "batch", "index"]
    with open(path, "w") as fh:
        for i in range(n):
            topic = rng.choice(words)
            q = f"what is {topic} {i}"
            p = " ".join([topic] + [rng.choice(words) for _ in range(rng.randint(20, 120))])
            negs = [" ".join(rng.choice(words) for _ in range(rng.randint(20, 120))) for _ in range(2)]
            fh.write(json.dumps({"query": q, "positive": p, "negatives": negs}) + "\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", default="train_synth.jsonl")
    ap.add_argument("--make-data", type=int, default=0)
    ap.add_argument("--batch-size", type=int, default=16)
    ap.add_argument("--max-steps", type=int, default=100)
    ap.add_argument("--lr", type=float, default=2e-5)
    ap.add_argument("--max-seq-length", type=int, default=256)
    ap.add_argument("--packed", action="store_true")
    ap.add_argument("--output-dir", default="output/script_run")
    args = ap.parse_args()

    from lset_b200.models.registry import detect_model_type
    from lset_b200.tokenization import load_tokenizer
    from lset_b200.train.data.dataset import EmbeddingDataset
    from lset_b200.train.engine import TrainingEngine

    if args.make_data:
        make_corpus(args.data, args.make_data)
    model_path = os.path.expanduser(args.model)
    tok = load_tokenizer(model_path)
    ds = EmbeddingDataset(args.data, tok, max_length=args.max_seq_length, num_hard_negatives=2)
    engine = TrainingEngine(detect_model_type(model_path), model_path, ds, batch_size=args.batch_size,
                            lr=args.lr, max_steps=args.max_steps, packed=args.packed, tokenizer=tok,
                            max_seq_length=args.max_seq_length, output_dir=args.output_dir)
    engine.train()


if __name__ == "__main__":
    main()
