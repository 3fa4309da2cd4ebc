"""Headline benchmark: contrastive training throughput of the Qwen3-0.6B embedder (bf16, packed
sequences, sharded data parallel), pairs/s and tokens/s on N GPUs of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Per GPU and step: 64 (query, positive) pairs, query lengths U[16,64], passage lengths U[128,512],
token ids U[0,151642), random N(0,0.02) weights, InfoNCE at temperature 0.02 over the global
in-batch negatives, AdamW, gradient clipping at 1.0. Weak scaling: the global batch grows with N.

Two timed regions of K steps each, after W warm-up steps, both bracketed by a barrier and a
device synchronisation and timed with CUDA events (max over ranks):
  * device: batches already resident on the GPU  -> "value" / "ms_per_step"
  * e2e:    ``TrainingEngine.train()``, the loop a user runs: DataLoader + collator on the host,
            pinned-memory H2D copy of the step's inputs, the step, and a device->host read of the
            step's global loss for the log line, every step -> "e2e"
Keys that describe the measurement rather than the workload are under "diagnostics".
Every step touches several GB of weights, optimizer state and activations, far more than the
126 MB L2, so no explicit L2 flush is needed between steps (stated in "config").
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

MODEL = dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
             num_attention_heads=16, num_key_value_heads=8, head_dim=128,
             max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1_000_000.0,
             tie_word_embeddings=True, attention_bias=False)
# The other training configurations of the comparison (selected with --config; the default is the
# headline one). "pairs" are per data-parallel rank.
MODEL_4B = dict(MODEL, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8)
MODEL_8B = dict(MODEL, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, tie_word_embeddings=False)
PRESETS = {
    "qwen3-0.6b": dict(
        model=MODEL, pairs=64, tp=1, negs=0, lora_r=0, q_len=(16, 64), d_len=(128, 512),
        metric="pairs/sec & tokens/sec, Qwen3-0.6B embed FSDP2 bf16, 1/2/4/8 B200, max over ranks",
        label="Qwen3-0.6B (28L, H1024, 16q/8kv heads, hd128, FFN3072, vocab 151936), random init"),
    "qwen3-4b-tp2": dict(
        model=MODEL_4B, pairs=32, tp=2, negs=0, lora_r=0, q_len=(16, 64), d_len=(256, 1024),
        metric="pairs/sec & tokens/sec, Qwen3-4B embed TP2 x sharded DP bf16, max over ranks",
        label="Qwen3-4B (36L, H2560, 32q/8kv heads, hd128, FFN9728, vocab 151936), random init"),
    "qwen3-4b": dict(
        model=MODEL_4B, pairs=32, tp=1, negs=0, lora_r=0, q_len=(16, 64), d_len=(256, 1024),
        metric="pairs/sec & tokens/sec, Qwen3-4B embed sharded DP bf16, max over ranks",
        label="Qwen3-4B (36L, H2560, 32q/8kv heads, hd128, FFN9728, vocab 151936), random init"),
    "qwen3-8b-lora": dict(
        model=MODEL_8B, pairs=16, tp=1, negs=3, lora_r=16, ac=True, q_len=(32, 32), d_len=(512, 512),
        metric="pairs/sec & tokens/sec, Qwen3-8B embed + LoRA r16, sharded DP bf16, 3 hard negatives, "
               "max over ranks",
        label="Qwen3-8B (36L, H4096, 32q/8kv heads, hd128, FFN12288, vocab 151936), random init, "
              "frozen base + LoRA r16 alpha 32 on q/k/v/o/gate/up/down"),
}
PAIRS_PER_GPU = 64
TOKEN_ID_MAX = 151642
TEMPERATURE = 0.02
LR = 2e-5
PUBLISHED_BASELINE = None  # the reference publishes no throughput number


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self._t = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self._t = threading.Thread(target=self._pump, daemon=True)
        self._t.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# data
# ----------------------------------------------------------------------------------------------
def make_samples(n_batches: int, rank: int, seed: int = 1234, pairs: int = PAIRS_PER_GPU,
                 negs: int = 0, q_len=(16, 64), d_len=(128, 512)):
    """Pre-tokenised samples: ``n_batches * pairs`` (query, positive[, negatives]) dicts for one
    data-parallel rank."""
    import torch

    gen = torch.Generator().manual_seed(seed + 7919 * rank)

    def seq(lo, hi):
        n = int(torch.randint(lo, hi + 1, (1,), generator=gen))
        return {"input_ids": torch.randint(0, TOKEN_ID_MAX, (n,), generator=gen).tolist(),
                "attention_mask": [1] * n}

    out = []
    for _ in range(n_batches * pairs):
        item = {"query": seq(*q_len), "positive": seq(*d_len)}
        if negs:
            item["negatives"] = [seq(*d_len) for _ in range(negs)]
        out.append(item)
    return out


class ListDataset:
    def __init__(self, items):
        self.items = items

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


def max_over_ranks(value: float, device) -> float:
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return value


def sum_over_ranks(value: float, device) -> float:
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())
    return value


def barrier_sync(device):
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize(device)


def _len_text(r):
    return str(r[0]) if r[0] == r[1] else f"U[{r[0]},{r[1]}]"


def result_line(impl, n_gpus, steps, warmup, ms, pairs, tokens, clocks, e2e, launches, diagnostics,
                preset=None):
    preset = preset or PRESETS["qwen3-0.6b"]
    pairs_s = pairs / (ms / 1e3)
    tp = preset["tp"]
    par = f"dp{n_gpus // tp}" + (f" x tp{tp}" if tp > 1 else "")
    line = {
        "metric": preset["metric"],
        "value": pairs_s, "unit": "pairs/s", "tokens_per_sec": tokens / (ms / 1e3),
        "n_gpus": n_gpus, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (pairs_s / PUBLISHED_BASELINE) if PUBLISHED_BASELINE else None,
        "dtype": "bf16", "data": "synthetic", "impl": impl,
        "config": {
            "model": preset["label"],
            "global_batch": pairs, "pairs_per_dp_rank": preset["pairs"],
            "hard_negatives_per_pair": preset["negs"],
            "seq_len": f"query {_len_text(preset['q_len'])}, passage {_len_text(preset['d_len'])}, "
                       "packed varlen stream (cu_seqlens)",
            "parallelism": par + (" (sharded optimizer/grad, ZeRO)" if n_gpus // tp > 1 else ""),
            "loss": "InfoNCE T=0.02, global in-batch negatives", "optimizer": "AdamW lr 2e-5, clip 1.0",
            "l2": "per-step working set (weights+optimizer+activations, several GB) exceeds the "
                  "126 MB L2; no explicit flush",
            "timing": "CUDA events on the launching stream, max over ranks, barrier+sync both sides",
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "diagnostics": diagnostics,
    }
    return line


# ----------------------------------------------------------------------------------------------
# this framework
# ----------------------------------------------------------------------------------------------
class TimedCollator:
    """Wraps a collator and marks the timed region of a ``train()`` loop from its collate calls (the
    DataLoader collates batch i right before step i): events are recorded at the calls ``first``
    and ``first + steps``, each with a barrier and a device synchronisation outside the region."""

    def __init__(self, inner, device=None, local_rank=0):
        self.inner, self.device, self.local_rank = inner, device, local_rank
        self.first = self.steps = None
        self.calls = 0
        self.h2d = 0
        self.tokens = []
        self.e0 = self.e1 = self.sampler = self.clocks = None

    def arm(self, first: int, steps: int, device, sample_clocks: bool = True):
        self.first, self.steps, self.device, self.calls = first, steps, device, 0
        self.sample_clocks = sample_clocks

    def __call__(self, batch):
        import torch

        i = self.calls
        self.calls += 1
        if self.first is not None and i == self.first:
            barrier_sync(self.device)
            if self.sample_clocks:
                self.sampler = ClockSampler(self.local_rank)
                self.sampler.start()
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        if self.first is not None and i == self.first + self.steps:
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e1.record()
            barrier_sync(self.device)
            if self.sampler is not None:
                self.clocks = self.sampler.stop()
        out = self.inner(batch)
        if self.first is not None and self.first <= i < self.first + self.steps:
            parts = [out[k] for k in ("query", "doc", "neg") if k in out]
            self.tokens.append(sum(int(p["input_ids"].numel()) for p in parts))
            self.h2d += sum(v.numel() * v.element_size() for p in parts for v in p.values()
                            if torch.is_tensor(v))
        return out


def run_ours(args):
    import contextlib

    import torch

    rank, local_rank, world = dist_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    from lset_b200.models import Qwen3Config
    from lset_b200.ops import _native as nv
    from lset_b200.train.data.collator import PackedCollator
    from lset_b200.train.engine import TrainingEngine, pin, to_device

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    nv.load()
    K, W = args.steps, args.warmup
    preset = PRESETS[args.config]
    tp, P = preset["tp"], preset["pairs"]
    if world % tp:
        raise SystemExit(f"--config {args.config} needs a multiple of {tp} GPUs")
    dp = world // tp

    class BenchCollator(PackedCollator):
        """Packed collator that also flattens a list of hard negatives per sample."""

        def __call__(self, batch):
            out = super().__call__(batch)
            if "negatives" in batch[0]:
                out["neg"] = self._batch([n for s in batch for n in s["negatives"]])
            return out

    lens = dict(q_len=preset["q_len"], d_len=preset["d_len"])
    # the end-to-end region runs the engine's own loop over this dataset (DataLoader, sampler,
    # collator, pinned-memory copies); every rank holds the same list, the sampler splits it
    e2e_steps = K + 2
    e2e_data = ListDataset(make_samples(e2e_steps * dp, 10_000, pairs=P, negs=preset["negs"], **lens))
    timed = TimedCollator(BenchCollator(), local_rank=local_rank)
    ac_mode = preset.get("ac_mode", "full")
    engine = TrainingEngine(
        "qwen3", None, dataset=e2e_data, dp_size=dp, tp_size=tp, batch_size=P, lr=LR,
        max_steps=10**9, grad_clip=1.0, temperature=TEMPERATURE, packed=True, log_interval=1,
        scheduler_type="constant", model_config=Qwen3Config(**preset["model"]),
        fused_projections=preset["lora_r"] == 0, collator=timed, async_tp=tp > 1,
        lora=preset["lora_r"] > 0, lora_r=max(1, preset["lora_r"]), lora_alpha=32.0,
        init_on_device=args.config != "qwen3-0.6b",
        fp8=args.fp8 is not None, fp8_recipe=args.fp8 or "rowwise",
        # the 8B model at this batch keeps several GB of activations per layer: recompute them
        activation_checkpoint=bool(preset.get("ac", False)), ac_mode=ac_mode,
        reshard_after_forward=args.reshard_after_forward)
    device = engine.device
    n_batches = W + K
    # ranks of one tensor-parallel group see the same batch
    samples = make_samples(n_batches, engine.dp_rank if tp > 1 else rank, pairs=P,
                           negs=preset["negs"], **lens)
    coll = BenchCollator()
    host = [pin(coll(samples[i * P:(i + 1) * P])) for i in range(n_batches)]
    tokens = [sum(int(b[k]["input_ids"].numel()) for k in ("query", "doc", "neg") if k in b)
              for b in host]
    # warm-up sees the largest batches, so the caching allocator has its blocks before timing
    order = sorted(range(n_batches), key=lambda i: -tokens[i])
    order = order[:W] + sorted(order[W:])
    host, tokens = [host[i] for i in order], [tokens[i] for i in order]

    for i in range(W):
        engine.train_step(host[i]).item()
    nv.check_status(device)

    # ---- device-timed region: inputs staged on the GPU beforehand
    staged = [to_device(host[W + i], device) for i in range(K)]
    barrier_sync(device)
    sampler = ClockSampler(local_rank)
    sampler.start()
    nv.reset_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t_host, wait0 = time.perf_counter(), engine.host_wait_s
    for i in range(K):
        engine.forward_backward(staged[i], True)
        engine.optimizer_step()
        engine.micro_step += 1
    # host time to enqueue a step, without the time it spent blocked on the run-ahead limit
    # (waiting for the GPU to finish the step before the previous one)
    wait_ms = (engine.host_wait_s - wait0) * 1e3 / K
    host_ms = (time.perf_counter() - t_host) * 1e3 / K - wait_ms
    e1.record()
    barrier_sync(device)
    clocks = sampler.stop()
    ms_dev = max_over_ranks(e0.elapsed_time(e1) / K, device)
    launches = nv.launches()
    tok_dev = sum_over_ranks(float(sum(tokens[W:W + K])) / K, device) / tp
    del staged

    # ---- end-to-end region: the engine's own train() loop. Every step: DataLoader + collate on
    # the host, pinned batch -> H2D, forward/backward/optimizer, loss read back for the log line.
    engine.max_steps = e2e_steps           # step 0 starts the loader; steps 1..K are timed
    engine.needs_dist_cleanup = False      # the process group is still needed for the reductions
    # One more untimed warm-up step, on the longest batch the loop is going to see (a dry pass
    # over the loader finds it: the order of an epoch depends on seed and epoch only, and train()
    # re-seeds it). A batch longer than all before it makes the caching allocator ask the driver
    # for new blocks, which on a shared host has stalled a step by several hundred milliseconds.
    if engine.sampler is not None:
        engine.sampler.set_epoch(engine.epoch)
    if engine._data_gen is not None:
        engine._data_gen.manual_seed(engine._data_seed + engine.epoch)
    longest, longest_tokens = None, -1
    for i, b in enumerate(engine.dataloader):
        if i >= e2e_steps:
            break
        n_tok = sum(int(b[k]["input_ids"].numel()) for k in ("query", "doc", "neg") if k in b)
        if n_tok > longest_tokens:
            longest, longest_tokens = b, n_tok
    if longest is not None:
        engine.train_step(longest).item()
        nv.check_status(device)
    timed.arm(1, K, device, sample_clocks=False)
    with contextlib.redirect_stdout(sys.stderr):   # the loop's own log lines
        last = engine.train()
    ms_e2e = max_over_ranks(timed.e0.elapsed_time(timed.e1) / K, device)
    nv.check_status(device)
    pairs = P * dp
    e2e = {"value": pairs / (ms_e2e / 1e3), "unit": "pairs/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": int(timed.h2d / K), "d2h_bytes_per_step": 4, "last_loss": last,
           "api": "lset_b200.train.engine.TrainingEngine.train() (DataLoader + collator + pinned "
                  "H2D + step + global loss read back and logged every step); one untimed warm-up "
                  "step on the longest batch of the loop before it"}
    if rank == 0:
        line = result_line("ours", world, K, W, ms_dev, pairs, tok_dev, clocks, e2e, launches,
                           {"host_enqueue_ms_per_step": round(host_ms, 2),
                            "host_blocked_on_gpu_ms_per_step": round(wait_ms, 2),
                            "fused_projections": preset["lora_r"] == 0,
                            "activation_checkpoint": ac_mode if preset.get("ac") else "off",
                            "parameter_sharding": ("layers sharded (ZeRO-3)" if engine.store.zero3
                                                   else "resident replica (ZeRO-2)"),
                            "memory": engine.store.memory_report(),
                            "native_library": str(nv.lib_path().name)}, preset)
        if args.fp8 is not None:
            # a side measurement, not the headline: linear layers on the 8-bit tensor-core GEMM
            line["dtype"] = f"fp8 ({args.fp8}: e4m3 operands, e5m2 gradients) in linear layers, bf16 elsewhere"
            line["vs_baseline"] = None
        print(json.dumps(line))
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# reference arm: the unmodified reference package from baseline/_ref, through its own engine
# ----------------------------------------------------------------------------------------------
def run_reference(args):
    preset = PRESETS[args.config]
    if preset["tp"] > 1:
        # The reference's tensor-parallel step was run once on these machines (2 x B200, TP2 x DP1, the
        # command below with --impl reference) and its own Triton code raised "an illegal memory
        # access was encountered" on rank 1. A GPU fault in the reference is not run a second time.
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference's tensor-parallel step faulted on these B200 machines (Triton Error "
                          "[CUDA]: an illegal memory access was encountered, TP2 x DP1 on 2 x B200); "
                          "its GPU code is not run again"}))
        return
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "lset")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/lset is not installed"}))
        return
    try:
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        sys.path.insert(0, ref_root)
        import lset  # noqa: F401
        from lset.train.data.packed_collator import PackedCollator as RefPacked
        from lset.train.engine import TrainingEngine as RefEngine
    except Exception as exc:  # pragma: no cover - depends on the box
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {exc!r}"[:300]}))
        return
    import torch.distributed as dist

    rank, local_rank, world = dist_env()
    K, W = args.steps, args.warmup
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)

    # The reference engine loads a checkpoint directory: write config.json and random N(0, 0.02)
    # weights once (rank 0) and let the other ranks wait for the marker file.
    model_dir = os.path.join(tempfile.gettempdir(),
                             f"lset_ref_{args.config}_{os.environ.get('MASTER_PORT', '0')}")
    marker = os.path.join(model_dir, "READY")
    if rank == 0 and not os.path.exists(marker):
        os.makedirs(model_dir, exist_ok=True)
        cfg = dict(preset["model"], model_type="qwen3", architectures=["Qwen3ForCausalLM"])
        with open(os.path.join(model_dir, "config.json"), "w") as fh:
            json.dump(cfg, fh)
        from lset.models import get_model_spec
        from safetensors.torch import save_file

        spec = get_model_spec("qwen3")
        torch.manual_seed(0)
        # built and filled on the GPU (host-side N(0, 0.02) of a multi-billion-parameter model takes
        # minutes), then written as the bf16 checkpoint the reference engine loads
        with torch.device(device):
            m = spec.model_cls(spec.config_cls.from_hf_json(os.path.join(model_dir, "config.json")))
        sd = {}
        for k, v in m.state_dict().items():
            t = v.detach()
            if t.dim() >= 2:
                t.normal_(0.0, 0.02)
            sd["model." + k] = t.to(torch.bfloat16).cpu().contiguous()
        save_file(sd, os.path.join(model_dir, "model.safetensors"))
        del m, sd
        torch.cuda.empty_cache()
        open(marker, "w").close()
    t_wait = time.time()
    while not os.path.exists(marker):
        time.sleep(0.5)
        if time.time() - t_wait > 600:
            print(json.dumps({"impl": "reference", "unavailable": "timed out waiting for weights"}))
            return

    n_batches = W + K + 1
    tp, P = preset["tp"], preset["pairs"]
    dp = max(1, world // tp)
    # with dp > 1 the reference's DistributedSampler gives each rank 1/dp of its dataset; the ranks
    # of one tensor-parallel group must see the same samples
    samples = make_samples(n_batches * dp, rank // tp if tp > 1 else rank, pairs=P,
                           negs=preset["negs"], q_len=preset["q_len"], d_len=preset["d_len"])
    tokens = []
    state = {"i": 0, "e0": None, "e1": None}
    if preset["negs"]:
        # the reference's packed collator takes one "negative" per sample; several hard negatives
        # per query are flattened into its "neg" batch with the reference's own packing routine
        from lset.train.data.packing import pack_sequences as ref_pack

        def inner(batch):
            return {"query": ref_pack([s["query"]["input_ids"] for s in batch]),
                    "doc": ref_pack([s["positive"]["input_ids"] for s in batch]),
                    "neg": ref_pack([n["input_ids"] for s in batch for n in s["negatives"]])}
    else:
        inner = RefPacked()

    def timing_collator(batch):
        # called by the engine's DataLoader right before each step (num_workers = 0)
        i = state["i"]
        if i == W:
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(device)
            state["sampler"] = ClockSampler(local_rank)
            state["sampler"].start()
            state["e0"] = torch.cuda.Event(enable_timing=True)
            state["e0"].record()
        if i == W + K:
            state["e1"] = torch.cuda.Event(enable_timing=True)
            state["e1"].record()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(device)
            state["clocks"] = state["sampler"].stop()
        out = inner(batch)
        if W <= i < W + K:
            parts = [out[k] for k in ("query", "doc", "neg") if k in out]
            tokens.append(sum(int(p["input_ids"].numel()) for p in parts))
            state["h2d"] = state.get("h2d", 0) + sum(
                v.numel() * v.element_size() for part in parts
                for v in part.values() if torch.is_tensor(v))
        state["i"] = i + 1
        return out

    class SeqDataset(ListDataset):
        pass

    try:
        engine = RefEngine(
            model_name="qwen3", model_path=model_dir, dataset=SeqDataset(samples), dp_size=dp,
            tp_size=tp, batch_size=P, lr=LR, max_steps=n_batches, grad_clip=1.0,
            temperature=TEMPERATURE, log_interval=10**9, packed=True, scheduler_type="constant",
            collator=timing_collator, lora=preset["lora_r"] > 0, lora_r=max(1, preset["lora_r"]),
            lora_alpha=32.0, activation_checkpoint=bool(preset.get("ac", False)),
            ac_mode=preset.get("ac_mode", "full"))
        # keep the batches in order (the stock DataLoader shuffles; order does not change the work)
        engine.train()
    except Exception as exc:  # pragma: no cover - depends on the box
        print(json.dumps({"impl": "reference", "unavailable": f"reference run failed: {exc!r}"[:400]}))
        return
    ms = state["e0"].elapsed_time(state["e1"]) / K
    if world > 1 and not dist.is_initialized():
        # the reference engine destroys the process group at the end of train(); reduce via files
        ms_all = _file_allreduce(ms, rank, world, "ms", max)
        tok_all = _file_allreduce(float(sum(tokens)) / K, rank, world, "tok", sum)
    else:
        ms_all, tok_all = ms, float(sum(tokens)) / K
    pairs = P * dp
    if tp > 1:
        tok_all /= tp   # every rank of a tensor-parallel group counted the same tokens
    e2e = {"value": pairs / (ms_all / 1e3), "unit": "pairs/s", "ms_per_step": ms_all,
           "h2d_bytes_per_step": int(state.get("h2d", 0) / K), "d2h_bytes_per_step": 4,
           "api": "lset.train.engine.TrainingEngine.train() (stock loop: .to(device) + loss.item() per step)"}
    if rank == 0:
        line = result_line("reference", world, K, W, ms_all, pairs, tok_all, state.get("clocks"), e2e,
                           None, {"note": "timed region = steps W..W+K-1 of the reference's own "
                                          "train() loop, marked from its DataLoader collate calls",
                                  "activation_checkpoint":
                                      preset.get("ac_mode", "full") if preset.get("ac") else "off"},
                           preset)
        line.pop("gpu_launches")
        print(json.dumps(line))


def _file_allreduce(value, rank, world, tag, op):
    d = os.path.join(tempfile.gettempdir(), f"lset_bench_{os.environ.get('MASTER_PORT', '0')}_{tag}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, f"{rank}.txt"), "w") as fh:
        fh.write(repr(float(value)))
    t0 = time.time()
    while time.time() - t0 < 120:
        try:
            vals = [float(open(os.path.join(d, f"{r}.txt")).read()) for r in range(world)]
            return op(vals)
        except (OSError, ValueError):
            time.sleep(0.2)
    return value


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=sorted(PRESETS), default="qwen3-0.6b")
    ap.add_argument("--fp8", choices=["tensorwise", "rowwise", "rowwise_with_gw_hp"], default=None,
                    help="side measurement: FP8 linear layers (the headline number is bf16)")
    ap.add_argument("--reshard-after-forward", action="store_true",
                    help="side measurement: shard the layers' parameters and gradients as well "
                         "(ZeRO-3); the headline keeps the resident bf16 replica")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
