"""Worker for engine-level multi-GPU equivalence tests (one rank per GPU under torch.distributed.run).

    mgpu_engine_worker.py OUT DP TP STEPS [zero3] [async_tp] [no_tp_runner]

Trains a small Qwen3 embedder for STEPS optimizer steps on a fixed global batch sequence (16 pairs
per step, split over the DP ranks; the ranks of one tensor-parallel group see the same pairs) and
writes, from rank 0, the global losses, the gradient norms, a fingerprint of the final master
weights and the per-rank bytes held in parameters, gradients and optimizer state."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lset_b200.models import Qwen3Config  # noqa: E402
from lset_b200.ops import _native as nv  # noqa: E402
from lset_b200.tasks.bi_encoder import global_loss_value  # noqa: E402
from lset_b200.train.data.collator import PackedCollator  # noqa: E402
from lset_b200.train.data.dataset import SyntheticPairDataset  # noqa: E402
from lset_b200.train.engine import TrainingEngine  # noqa: E402

GLOBAL_PAIRS = 16


def main():
    out_path, dp, tp, steps = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    flags = set(sys.argv[5:])
    rank = int(os.environ.get("RANK", 0))
    cfg = Qwen3Config(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=3,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    if "no_tp_runner" in flags:   # tensor-parallel blocks op by op instead of one native call each
        from lset_b200.ops.runtime_options import configure

        configure(tp_block_runner=False)
    per = GLOBAL_PAIRS // dp
    eng = TrainingEngine("qwen3", None, None, dp_size=dp, tp_size=tp, batch_size=per, lr=1e-3,
                         packed=True, model_config=cfg, fused_projections=True, log_interval=0,
                         grad_clip=1.0, scheduler_type="constant", async_tp="async_tp" in flags,
                         reshard_after_forward="zero3" in flags)
    ds = SyntheticPairDataset(GLOBAL_PAIRS * steps, 2048, (8, 24), (40, 200), seed=11)
    coll = PackedCollator()
    losses, norms = [], []
    for s in range(steps):
        base = s * GLOBAL_PAIRS + eng.dp_rank * per
        loss = eng.train_step(coll([ds[i] for i in range(base, base + per)]))
        losses.append(float(global_loss_value(loss, eng.dp_group)))
        norms.append(float(eng.optimizer.grad_norm()))
    nv.check_status()
    torch.cuda.synchronize()
    masters = dict(eng.store.named_master_tensors())      # full tensors over dp (a collective)
    if tp > 1:
        from lset_b200.dist.tp import unshard

        for name, p in eng.model.named_parameters():
            if hasattr(p, "_tp_meta") and name in masters:
                masters[name] = unshard(masters[name], p._tp_meta, eng.tp_group)
    finger = {n: [float(t.double().sum()), float(t.double().pow(2).sum())]
              for n, t in sorted(masters.items())}
    mem = eng.store.memory_report() if hasattr(eng.store, "memory_report") else {}
    if rank == 0:
        with open(out_path, "w") as f:
            from lset_b200.ops import block as block_ops

            json.dump({"losses": losses, "norms": norms, "fingerprint": finger, "memory": mem,
                       "symm": bool(eng.store.use_symm), "runner_calls": dict(block_ops.calls)}, f)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
