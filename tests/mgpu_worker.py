"""Worker for the multi-GPU tests (launched with torch.distributed.run, one rank per GPU).

Runs a few optimizer steps of a small Qwen3 embedder through the engine and writes, from rank 0,
the per-step global losses, gradient norms and a fingerprint of the final parameters."""
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


def main():
    out_path, steps = sys.argv[1], int(sys.argv[2])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cfg = Qwen3Config(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=3,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    eng = TrainingEngine("qwen3", None, None, dp_size=world, batch_size=8, lr=1e-3, packed=True,
                         model_config=cfg, fused_projections=True, log_interval=0, grad_clip=1.0,
                         scheduler_type="constant")
    ds = SyntheticPairDataset(8 * world * steps, 2048, (8, 24), (40, 200), seed=11)
    coll = PackedCollator()
    losses, norms = [], []
    for s in range(steps):
        base = (s * world + rank) * 8
        loss = eng.train_step(coll([ds[i] for i in range(base, base + 8)]))
        losses.append(float(global_loss_value(loss, eng.dp_group)))
        norms.append(float(eng.optimizer.grad_norm()))
    nv.check_status()
    torch.cuda.synchronize()
    fp = [float(g.flat_param.float().double().sum()) for g in eng.store.groups]
    fp2 = [float(g.flat_param.float().double().pow(2).sum()) for g in eng.store.groups]
    # every rank must hold identical parameters after the all-gather / push
    t = torch.tensor(fp + fp2, dtype=torch.float64, device=eng.device)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    if rank == 0:
        with open(out_path, "w") as fh:
            json.dump({"losses": losses, "norms": norms, "sum": fp, "sumsq": fp2,
                       "replicas_equal": bool(torch.equal(lo, hi)), "symm": eng.store.use_symm}, fh)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
