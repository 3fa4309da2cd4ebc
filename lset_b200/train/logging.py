"""Training logger: rank-0 console lines ``step=… k=v``, optional wandb, optional JSONL file, and
throughput accounting (pairs/s, tokens/s) that the engine actually feeds
(console format of lset/train/logging.py:25-38)."""
from __future__ import annotations

import json
import os
import time
from typing import Optional


class TrainLogger:
    def __init__(self, use_wandb: bool = False, project: str = "lset", config: Optional[dict] = None,
                 jsonl_path: Optional[str] = None, enabled: bool = True):
        self.enabled = enabled
        self._wandb = None
        self._jsonl = None
        if enabled and use_wandb:
            try:
                import wandb

                wandb.init(project=project, config=config or {})
                self._wandb = wandb
            except Exception as exc:  # pragma: no cover - optional dependency
                print(f"wandb unavailable ({exc}); console logging only")
        if enabled and jsonl_path:
            os.makedirs(os.path.dirname(jsonl_path) or ".", exist_ok=True)
            self._jsonl = open(jsonl_path, "a")
        self._t0 = time.time()
        self._samples = 0
        self._tokens = 0

    def log(self, step: int, metrics: dict) -> None:
        if not self.enabled:
            return
        parts = [f"step={step}"]
        for k, v in metrics.items():
            parts.append(f"{k}={v:.4f}" if isinstance(v, float) else f"{k}={v}")
        print(" ".join(parts), flush=True)
        if self._wandb is not None:
            self._wandb.log(metrics, step=step)
        if self._jsonl is not None:
            self._jsonl.write(json.dumps({"step": step, **metrics}) + "\n")
            self._jsonl.flush()

    def update_throughput(self, num_samples: int, num_tokens: int = 0) -> dict:
        self._samples += num_samples
        self._tokens += num_tokens
        dt = max(1e-9, time.time() - self._t0)
        return {"samples_per_sec": self._samples / dt, "tokens_per_sec": self._tokens / dt}

    def reset_throughput(self) -> None:
        self._t0, self._samples, self._tokens = time.time(), 0, 0

    def finish(self) -> None:
        if self._wandb is not None:
            self._wandb.finish()
        if self._jsonl is not None:
            self._jsonl.close()
            self._jsonl = None
