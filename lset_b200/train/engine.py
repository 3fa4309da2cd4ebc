"""Training engine: model construction, sharded runtime, task, optimizer, data loading, the loop.

Constructor arguments follow the reference's engine (lset/train/engine.py:45-140) so existing
callers keep working; additions are keyword-only in spirit: ``model_config`` (build a randomly
initialised model instead of loading a checkpoint), ``pooling`` / ``padding_side`` overrides,
``fused_projections``, ``length_sorted``, ``learnable_temperature``, ``weight_decay``,
``step_timeout_s``, ``device``.

One optimizer step (``train_step``):
  host batch -> device (non-blocking copies from pinned memory) -> task forward (queries, documents
  and negatives share one packed forward) -> backward (weight gradients accumulate in fp32 flat
  buffers; each layer's buffer is reduce-scattered as soon as its backward is done) -> on the
  accumulation boundary: device-side global-norm clipping + fused AdamW + parameter all-gather.
Nothing in the step synchronises with the host; the loss is read back only when it is logged.
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Optional

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, DistributedSampler

from ..dist.sharded import ParamStore, ShardedAdamW
from ..models import get_model_spec
from ..models.layers import init_normal_
from ..tasks.bi_encoder import BiEncoderTask, global_loss_value
from .checkpoint import latest_checkpoint, load_checkpoint, load_extra, save_checkpoint
from .logging import TrainLogger
from .scheduler import build_scheduler
from .watchdog import maybe_fail
from ..utils.tracing import PhaseTimer


def to_device(obj, device, non_blocking: bool = True):
    if torch.is_tensor(obj):
        return obj.to(device, non_blocking=non_blocking)
    if isinstance(obj, dict):
        return {k: to_device(v, device, non_blocking) for k, v in obj.items()}
    return obj


def pin(obj):
    """Pinned-memory copy of every tensor in a (nested) batch; identity without CUDA."""
    if not torch.cuda.is_available():
        return obj
    if torch.is_tensor(obj):
        return obj.pin_memory()
    if isinstance(obj, dict):
        return {k: pin(v) for k, v in obj.items()}
    return obj


def batch_tokens(batch: dict) -> int:
    n = 0
    for key in ("query", "doc", "neg"):
        b = batch.get(key)
        if b is None:
            continue
        n += int(b["attention_mask"].sum()) if "attention_mask" in b else int(b["input_ids"].numel())
    return n


def batch_bytes(obj) -> int:
    if torch.is_tensor(obj):
        return obj.numel() * obj.element_size()
    if isinstance(obj, dict):
        return sum(batch_bytes(v) for v in obj.values())
    return 0


def _init_process_group(backend: str, rank: int, world: int) -> None:
    """``init_process_group`` from the launcher's environment. A worker group restarted by the
    launcher (``--max-restarts``) meets on the same store as the attempt before it; its rendezvous
    keys are put under a prefix of their own so that addresses left by dead workers are not read."""
    restart = int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0"))
    if restart == 0 or "MASTER_ADDR" not in os.environ or "MASTER_PORT" not in os.environ:
        dist.init_process_group(backend)
        return
    from datetime import timedelta

    store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), world,
                          is_master=False, timeout=timedelta(seconds=300))
    dist.init_process_group(backend, store=dist.PrefixStore(f"attempt{restart}", store), rank=rank,
                            world_size=world)


class TrainingEngine:
    def __init__(self, model_name: str, model_path: Optional[str], dataset, dp_size: int = 1,
                 tp_size: int = 1, batch_size: int = 8, lr: float = 1e-5, max_steps: int = 1000,
                 grad_clip: float = 1.0, temperature: float = 0.02, matryoshka_dims=None,
                 log_interval: int = 10, packed: bool = False, use_grad_cache: bool = False,
                 gc_chunk_size: Optional[int] = 16, gc_token_budget: Optional[int] = None,
                 gc_selective_keep: float = 1.0, gradient_accumulation_steps: int = 1,
                 save_steps: int = 0, output_dir: str = "./output", resume_from: Optional[str] = None,
                 scheduler_type: str = "cosine", warmup_steps: int = 0, use_wandb: bool = False,
                 wandb_project: str = "lset", use_label_matrix: bool = False, collator=None,
                 lora: bool = False, lora_r: int = 8, lora_alpha: float = 16.0,
                 lora_dropout: float = 0.0, lora_targets=None, qlora: bool = False,
                 qlora_block_size: int = 64, fp8: bool = False, fp8_recipe: str = "rowwise",
                 attn_backend: str = "auto", cuda_graph: bool = False,
                 cuda_graph_token_budget: Optional[int] = None, top_k: Optional[int] = None,
                 cascade: bool = False, cascade_d_small: int = 64, cascade_K_prime: int = 256,
                 activation_checkpoint: bool = False, ac_mode: str = "selective",
                 ac_ratio: float = 1.0, async_tp: bool = False,
                 # extensions
                 model_config=None, pooling: str = "auto", padding_side: str = "auto",
                 fused_projections: bool = False, length_sorted: bool = False,
                 learnable_temperature: bool = False, weight_decay: float = 0.01,
                 step_timeout_s: float = 0.0, device: Optional[str] = None, seed: int = 42,
                 max_seq_length: int = 512, tokenizer=None, num_workers: int = 0,
                 jsonl_log: bool = False, init_std: float = 0.02, init_on_device: bool = False,
                 max_inflight_steps: int = 2, reshard_after_forward: bool = False):
        if cuda_graph:
            from .cuda_graph import validate_cuda_graph_config

            validate_cuda_graph_config(packed, use_grad_cache, compile_model=False,
                                       token_budget=cuda_graph_token_budget)
        if fp8 and (lora or qlora):
            raise ValueError("FP8 training + LoRA/QLoRA is not supported")
        if qlora and tp_size > 1:
            raise ValueError("QLoRA + tensor parallelism is not supported")

        self.dp_size, self.tp_size = dp_size, tp_size
        self.batch_size, self.max_steps = batch_size, max_steps
        self.grad_clip, self.log_interval = grad_clip, log_interval
        self.grad_accum_steps = max(1, gradient_accumulation_steps)
        self.save_steps, self.output_dir, self.resume_from = save_steps, output_dir, resume_from
        self.use_label_matrix = use_label_matrix
        self.use_grad_cache = use_grad_cache
        self.packed = packed
        self.use_lora = lora or qlora
        self.step_timeout_s = step_timeout_s
        self.save_timeout_s = max(600.0, 20.0 * float(step_timeout_s or 0.0))
        self.needs_dist_cleanup = False

        # ---------------------------------------------------------------- process group / device
        world = dp_size * tp_size
        self.rank = int(os.environ.get("RANK", 0))
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        use_cuda = torch.cuda.is_available() and device != "cpu"
        if world > 1 and not dist.is_initialized():
            _init_process_group("nccl" if use_cuda else "gloo", self.rank, world)
            self.needs_dist_cleanup = True
        if use_cuda:
            torch.cuda.set_device(self.local_rank)
            self.device = torch.device("cuda", self.local_rank)
        else:
            self.device = torch.device("cpu")
        self.compute_dtype = torch.bfloat16 if use_cuda else torch.float32
        torch.manual_seed(seed)

        # ---------------------------------------------------------------- mesh
        self.mesh = None
        self.dp_group = self.tp_group = None
        self.dp_rank, self.tp_rank = self.rank, 0
        if world > 1:
            from ..dist.mesh import build_mesh

            self.mesh = build_mesh(dp_size, tp_size, device_type="cuda" if use_cuda else "cpu")
            if tp_size > 1:
                self.dp_group = self.mesh["dp"].get_group()
                self.tp_group = self.mesh["tp"].get_group()
                self.dp_rank = self.mesh["dp"].get_local_rank()
                self.tp_rank = self.mesh["tp"].get_local_rank()

        # ---------------------------------------------------------------- model
        spec = get_model_spec(model_name)
        self.spec = spec
        if model_config is None:
            model_config = spec.config_cls.from_hf_json(str(Path(model_path) / "config.json"))
        self.model_config = model_config
        has_weights = model_path is not None and (
            any(Path(model_path).glob("*.safetensors")) or any(Path(model_path).glob("pytorch_model*.bin")))
        if has_weights:
            model = spec.model_cls(model_config, fused_projections=fused_projections)
            state = spec.weight_converter(model_path, fused_projections=fused_projections)
            model.load_state_dict(state, strict=True)
        else:
            # Random initialisation: on the host by default (bit-identical start on CPU and GPU
            # runs); init_on_device builds and fills the model on the target device, which is what
            # multi-billion-parameter models need (host-side init takes minutes per rank).
            with torch.device(self.device if init_on_device else "cpu"):
                model = spec.model_cls(model_config, fused_projections=fused_projections)
            init_normal_(model, init_std)
        if self.use_lora:
            from .lora import apply_lora, apply_qlora

            if qlora:
                apply_qlora(model, r=lora_r, alpha=lora_alpha, dropout=lora_dropout,
                            target_modules=lora_targets, block_size=qlora_block_size)
            else:
                apply_lora(model, r=lora_r, alpha=lora_alpha, dropout=lora_dropout,
                           target_modules=lora_targets)
        if fp8:
            from .quantization.fp8 import apply_fp8_training

            apply_fp8_training(model, recipe=fp8_recipe)
        if tp_size > 1:
            from ..dist.tp import apply_tp

            # async_tp: token-sharded residual stream with the all-gather / reduce-scatter fused
            # into the projection GEMMs over peer memory (decoder families, no LoRA adapters);
            # otherwise the Megatron all-reduce scheme.
            # FP8 linear layers keep their own forward, so they run under the all-reduce scheme.
            sp = bool(async_tp) and not self.use_lora and not fp8 and hasattr(model, "_sp")
            apply_tp(model, self.tp_group, spec.tp_plan_fn(
                model_config, use_sequence_parallel=sp, use_lora=self.use_lora,
                fused_projections=fused_projections), sequence_parallel=sp)
        if activation_checkpoint:
            from ..dist.activation_checkpoint import apply_activation_checkpointing

            apply_activation_checkpointing(model, mode=ac_mode, ratio=ac_ratio)
        self.model = model

        # ---------------------------------------------------------------- task
        pool_name = spec.default_pooling if pooling in (None, "auto") else pooling
        self.padding_side = spec.default_padding_side if padding_side in (None, "auto") else padding_side
        self.task = BiEncoderTask(
            pooling=pool_name, temperature=temperature, matryoshka_dims=matryoshka_dims, top_k=top_k,
            learnable_scale=learnable_temperature, cascade=cascade, cascade_d_small=cascade_d_small,
            cascade_K_prime=cascade_K_prime, dp_group=self.dp_group)
        if spec.post_pooling_fn is not None and model_path is not None:
            proj = spec.post_pooling_fn(model_path)
            if proj is not None:
                self.task.set_post_pooling(proj.to(self.device, self.compute_dtype))
        self.task.to(self.device)

        # ---------------------------------------------------------------- sharded runtime + optimizer
        self.store = ParamStore(model, dp_group=self.dp_group if world > 1 else None,
                                compute_dtype=self.compute_dtype, device=self.device,
                                tp_group=self.tp_group,
                                reshard_after_forward=reshard_after_forward)
        if self.task.logit_scale is not None:
            self.task_store = ParamStore(self.task, layer_modules=[], dp_group=None,
                                         compute_dtype=torch.float32, device=self.device)
        else:
            self.task_store = None
        self.optimizer = ShardedAdamW(self.store, lr=lr, weight_decay=weight_decay,
                                      grad_clip=grad_clip)
        self.task_optimizer = (ShardedAdamW(self.task_store, lr=lr, weight_decay=0.0)
                               if self.task_store is not None else None)
        self.scheduler = build_scheduler(self.optimizer, scheduler_type, warmup_steps,
                                         max(1, max_steps // self.grad_accum_steps))
        self.grad_cache = None
        if use_grad_cache:
            from .grad_cache import GradCacheWrapper

            self.grad_cache = GradCacheWrapper(
                self.task, chunk_size=gc_chunk_size, token_budget=gc_token_budget,
                selective_keep=gc_selective_keep, store=self.store)

        # ---------------------------------------------------------------- logging
        is_rank0 = self.rank == 0
        self.logger = TrainLogger(use_wandb=use_wandb and is_rank0, project=wandb_project,
                                  jsonl_path=(os.path.join(output_dir, "metrics.jsonl")
                                              if jsonl_log and is_rank0 else None),
                                  enabled=is_rank0)

        # ---------------------------------------------------------------- data
        self.dataset = dataset
        self._data_gen, self._data_seed, self._batch_in_epoch = None, seed, 0
        self.collator = collator if collator is not None else self._pick_collator(
            dataset, tokenizer, max_seq_length, length_sorted)
        self.sampler = None
        self.dataloader = None
        if dataset is not None:
            if dp_size > 1:
                self.sampler = DistributedSampler(dataset, num_replicas=dp_size, rank=self.dp_rank,
                                                  shuffle=True, seed=seed)
            gen = torch.Generator().manual_seed(seed)
            self._data_gen, self._data_seed = gen, seed
            self.dataloader = DataLoader(
                dataset, batch_size=batch_size, sampler=self.sampler,
                shuffle=self.sampler is None, collate_fn=self.collator, drop_last=True,
                num_workers=num_workers, pin_memory=use_cuda, generator=gen)
        self.micro_step = 0
        self.max_inflight_steps = max_inflight_steps
        self._inflight = []
        self.host_wait_s = 0.0
        self.epoch = 0
        # per-phase device timing (h2d / forward_backward / optimizer); LSET_B200_PROFILE=1 enables it
        self.timer = PhaseTimer(enabled=os.environ.get("LSET_B200_PROFILE", "0") == "1")
        self.watchdog = None
        if step_timeout_s and step_timeout_s > 0:
            from .watchdog import StepWatchdog

            self.watchdog = StepWatchdog(step_timeout_s)
        self.heartbeat = None
        if step_timeout_s and step_timeout_s > 0 and world > 1 and dist.is_initialized():
            from ..dist.health import RankHeartbeat

            try:
                store = dist.distributed_c10d._get_default_store()
                self.heartbeat = RankHeartbeat(store, dist.get_rank(), dist.get_world_size(),
                                               stale_s=max(2.0, step_timeout_s / 2))
                self.heartbeat.start()
            except Exception as exc:  # pragma: no cover - store not reachable
                print(f"[lset_b200] heartbeat disabled: {exc}")

    # ------------------------------------------------------------------ helpers
    def _pick_collator(self, dataset, tokenizer, max_seq_length, length_sorted):
        from .data.collator import (EmbeddingCollator, LeftPadCollator, PackedCollator,
                                    RightPadCollator)

        if dataset is None:
            return None
        if hasattr(dataset, "format"):  # text dataset -> label-matrix collator
            tok = tokenizer if tokenizer is not None else getattr(dataset, "tokenizer", None)
            self.use_label_matrix = True
            return EmbeddingCollator(tok, max_length=max_seq_length, packed=self.packed,
                                     length_sorted=length_sorted, padding_side=self.padding_side)
        if self.packed:
            return PackedCollator()
        return LeftPadCollator(0) if self.padding_side == "left" else RightPadCollator(0)

    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.store.set_requires_gradient_sync(flag)

    # ------------------------------------------------------------------ one micro-step
    def forward_backward(self, batch: dict, is_boundary: bool = True):
        """Forward + backward of one micro-batch (moved to the device if it is not there). Returns the detached local
        loss share (sum over ranks = global loss)."""
        ga = self.grad_accum_steps
        batch = to_device(batch, self.device)  # no-op for tensors that are already there
        self.store.set_requires_gradient_sync(is_boundary)
        q, d, n = batch["query"], batch["doc"], batch.get("neg")
        labels = batch.get("labels") if self.use_label_matrix else None
        scores = batch.get("scores") if self.use_label_matrix else None
        if self.grad_cache is not None:
            loss = self.grad_cache(self.model, q, d, neg_batch=n, labels=labels, scores=scores,
                                   is_ga_boundary=is_boundary, grad_output=1.0 / ga)
        else:
            out = self.task(self.model, q, d, n, labels=labels, scores=scores,
                            pos_qi=batch.get("pos_qi"), pos_di=batch.get("pos_di"),
                            pos_counts=batch.get("pos_counts"))
            loss = out["loss"]
            (loss / ga if ga > 1 else loss).backward()
            loss = loss.detach()
        self.store.finish_backward()
        if self.task_store is not None:
            self.task_store.finish_backward()
        return loss

    def optimizer_step(self) -> None:
        self.optimizer.step()
        if self.task_optimizer is not None:
            self.task_optimizer.step()
            self.task_optimizer.zero_grad()
        self.scheduler.step()
        self.optimizer.zero_grad()
        self._limit_run_ahead()
        if self.device.type == "cuda":
            from ..ops import _native as nv

            nv.poll_status(self.device)  # a kernel that gave up a bounded wait fails the run loudly

    def _limit_run_ahead(self) -> None:
        """Keep the host at most ``max_inflight_steps`` optimizer steps ahead of the GPU. A host
        that queues many steps ahead makes the caching allocator hold the blocks of all of them
        (side-stream frees are deferred until their events complete) and fall back to fresh device
        allocations, which are slow once peer access to many GPUs is enabled. Waiting on the event
        of an older step costs nothing while the GPU is the bottleneck."""
        if self.device.type != "cuda" or self.max_inflight_steps <= 0:
            return
        ev = torch.cuda.Event()
        ev.record()
        self._inflight.append(ev)
        t0 = time.perf_counter()
        while len(self._inflight) > self.max_inflight_steps:
            self._inflight.pop(0).synchronize()
        self.host_wait_s += time.perf_counter() - t0   # host time spent waiting for the GPU

    def train_step(self, batch: dict):
        """One micro-step from a host batch: H2D copy, forward/backward and, on the accumulation
        boundary, the optimizer update. Returns the local loss share as a device tensor."""
        if self.watchdog is not None:
            self.watchdog.beat()
        if self.heartbeat is not None:
            self.heartbeat.check_peers()  # a dead peer is noticed before the next collective
        with self.timer.phase("h2d"):
            batch = to_device(batch, self.device)
        boundary = (self.micro_step + 1) % self.grad_accum_steps == 0
        with self.timer.phase("forward_backward"):
            loss = self.forward_backward(batch, boundary)
        if boundary:
            with self.timer.phase("optimizer"):
                self.optimizer_step()
        self.micro_step += 1
        return loss

    # ------------------------------------------------------------------ loop
    def train(self):
        start, skip = 0, 0
        resume = self.resume_from
        if resume == "auto":
            resume = latest_checkpoint(self.output_dir)
        if resume:
            start = load_checkpoint(self.model, self.optimizer, resume, store=self.store)
            extra = load_extra(resume)
            if extra is not None:
                self.scheduler.load_state_dict(extra.get("scheduler", self.scheduler.state_dict()))
                self.epoch = int(extra.get("epoch", 0))
                if "rng" in extra:
                    torch.set_rng_state(extra["rng"])
                if "cuda_rng" in extra and self.device.type == "cuda":
                    torch.cuda.set_rng_state(extra["cuda_rng"].cpu(), self.device)
                skip = int(extra.get("batch_in_epoch", 0))
                if self.task_store is not None and "task" in extra:
                    self.task.load_state_dict(extra["task"])
                    self.task_store.load_master(extra["task"])
                    self.task_optimizer.load_state_dict(extra["task_optimizer"])
            self.micro_step = start
            if self.watchdog is not None:
                self.watchdog.beat()       # loading a checkpoint is not idle time
        step = start
        last_loss = None
        self.logger.reset_throughput()
        t_last, steps_last = time.time(), step
        if self.watchdog is not None:
            self.watchdog.start()
        try:
            while step < self.max_steps:
                if self.sampler is not None:
                    self.sampler.set_epoch(self.epoch)
                if self._data_gen is not None:
                    # the order of an epoch depends on (seed, epoch) only, so that a resumed run
                    # can continue in the middle of one
                    self._data_gen.manual_seed(self._data_seed + self.epoch)
                batches = iter(self.dataloader)
                made_progress = skip > 0
                for _ in range(skip):          # resume: batches this epoch had already consumed
                    if next(batches, None) is None:
                        break
                self._batch_in_epoch, skip = skip, 0
                # The next batch is collated (and pinned) right after this step's kernels are
                # enqueued, before the loss is read back: host-side batch preparation runs under
                # the GPU's work instead of in the gap between two steps.
                batch = next(batches, None)
                while batch is not None:
                    if step >= self.max_steps:
                        break
                    made_progress = True
                    self._batch_in_epoch += 1
                    n_pairs = self._batch_pairs(batch)
                    n_tok = batch_tokens(batch)
                    maybe_fail(step, self.rank)      # host-side fault injection (off unless asked for)
                    loss = self.train_step(batch)
                    batch = next(batches, None) if step + 1 < self.max_steps else None
                    tp = self.logger.update_throughput(n_pairs * self.dp_size, n_tok * self.dp_size)
                    if self.log_interval and step % self.log_interval == 0:
                        value = float(global_loss_value(loss, self.dp_group))
                        last_loss = value
                        now = time.time()
                        self.logger.log(step, {
                            "loss": value, "lr": self.scheduler.get_last_lr()[0],
                            "pairs_per_sec": tp["samples_per_sec"],
                            "tokens_per_sec": tp["tokens_per_sec"],
                            "step_ms": 1e3 * (now - t_last) / max(1, step - steps_last)})
                        t_last, steps_last = now, step
                    if self.save_steps and (step + 1) % self.save_steps == 0:
                        self.save(step + 1)
                    step += 1
                if step < self.max_steps:
                    self.epoch += 1
                    self._batch_in_epoch = 0
                if not made_progress:
                    if step == start and self.rank == 0:
                        print(f"[lset_b200] no full batch of {self.batch_size} samples per rank in "
                              f"the dataset ({len(self.dataset)} samples): nothing to train on")
                    break
        finally:
            if self.watchdog is not None:
                self.watchdog.stop()
            if self.heartbeat is not None:
                self.heartbeat.stop()
            self.logger.finish()
            if self.needs_dist_cleanup and dist.is_initialized():
                dist.destroy_process_group()
        return last_loss

    def save(self, step: int) -> str:
        if self.device.type == "cuda":
            from ..ops import _native as nv

            # a kernel that gave up a bounded wait leaves a non-zero status word: such a state is
            # never written out (synchronising read; every rank checks before the collectives)
            nv.check_status(self.device)
        if self.watchdog is None:
            return self._save(step)
        # gathering and writing a large model takes longer than a step: the save runs under its
        # own, larger idle limit instead of tripping the step watchdog on every attempt
        with self.watchdog.extended(self.save_timeout_s):
            return self._save(step)

    def _save(self, step: int) -> str:
        extra = {"scheduler": self.scheduler.state_dict(), "epoch": self.epoch,
                 "rng": torch.get_rng_state(), "micro_step": self.micro_step,
                 "batch_in_epoch": self._batch_in_epoch}
        if self.device.type == "cuda":     # dropout masks on the GPU come from its own generator
            extra["cuda_rng"] = torch.cuda.get_rng_state(self.device)
        if self.task_store is not None:    # the learnable temperature lives outside the model
            extra["task"] = {k: v.detach().cpu() for k, v in self.task.state_dict().items()}
            extra["task_optimizer"] = self.task_optimizer.state_dict()
        return save_checkpoint(self.model, self.optimizer, step, self.output_dir, store=self.store,
                               extra=extra)

    @staticmethod
    def _batch_pairs(batch: dict) -> int:
        q = batch["query"]
        if "cu_seqlens" in q:
            return int(q.get("num_sequences", q["cu_seqlens"].numel() - 1))
        return int(q["input_ids"].shape[0])
