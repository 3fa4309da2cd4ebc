"""Worker (torch.distributed.run, one rank per GPU): cross-rank fused InfoNCE against the fp32
reference built from an NCCL all-gather. Two calls per shape, so buffer reuse is covered."""
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lset_b200.dist.xrank_loss import cross_rank_infonce, supported  # noqa: E402
from lset_b200.ops import _native as nv  # noqa: E402


def main():
    out_path = sys.argv[1]
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    cases = []
    from lset_b200.ops import loss as loss_ops

    full_panel = (loss_ops.PANEL_BYTES, loss_ops.PANEL_MIN_COLS)
    for B, D in [(64, 1024), (264, 768), (1024, 256), (64, 1024)]:
        # small cases take the backward in one pass over every rank's passages; the 1024-row case
        # is made to walk four column panels per peer (the path of score matrices above the cap)
        loss_ops.PANEL_BYTES, loss_ops.PANEL_MIN_COLS = (256 * 1024, 256) if B == 1024 else full_panel
        for rep in range(2):
            torch.manual_seed(100 * rank + rep + B)
            q = F.normalize(torch.randn(B, D, device=dev), dim=-1).to(torch.bfloat16).requires_grad_()
            d = F.normalize(torch.randn(B, D, device=dev), dim=-1).to(torch.bfloat16).requires_grad_()
            assert supported(q, d)
            loss = cross_rank_infonce(q, d, 0.02)
            loss.backward()
            nv.check_status()
            # reference: gather everything, full fp32 loss; this rank's share and gradients
            qs = [torch.empty_like(q) for _ in range(world)]
            ds = [torch.empty_like(d) for _ in range(world)]
            dist.all_gather(qs, q.detach())
            dist.all_gather(ds, d.detach())
            Q = torch.cat(qs).float().requires_grad_()
            K = torch.cat(ds).float().requires_grad_()
            ce = F.cross_entropy(Q @ K.t() / 0.02, torch.arange(world * B, device=dev), reduction="none")
            (ce.sum() / (world * B)).backward()
            share = ce[rank * B:(rank + 1) * B].sum() / (world * B)
            dq_ref, dk_ref = Q.grad[rank * B:(rank + 1) * B], K.grad[rank * B:(rank + 1) * B]
            cases.append({
                "B": B, "D": D, "rep": rep,
                "loss_err": abs(loss.item() - share.item()) / max(1e-3, abs(share.item())),
                "dq_err": ((q.grad.float() - dq_ref).abs().max() / (dq_ref.abs().max() + 1e-9)).item(),
                "dk_err": ((d.grad.float() - dk_ref).abs().max() / (dk_ref.abs().max() + 1e-9)).item()})
    loss_ops.PANEL_BYTES, loss_ops.PANEL_MIN_COLS = full_panel
    # hard negatives through the task: every rank's block is [documents; negatives]
    from lset_b200.tasks.bi_encoder import BiEncoderTask

    task = BiEncoderTask(temperature=0.02)
    B, Bn, D = 64, 192, 512
    torch.manual_seed(7 + rank)
    q, d, n = (F.normalize(torch.randn(r, D, device=dev), dim=-1).to(torch.bfloat16).requires_grad_()
               for r in (B, B, Bn))
    loss = task.loss_from_embeddings(q, d, n)
    loss.backward()
    nv.check_status()

    def gathered(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.detach())
        return torch.cat(parts).float().requires_grad_()

    Q, Kd, Kn = gathered(q), gathered(d), gathered(n)
    logits = Q @ torch.cat([Kd, Kn]).t() / 0.02
    ce = F.cross_entropy(logits, torch.arange(world * B, device=dev), reduction="none")
    (ce.sum() / (world * B)).backward()
    share = ce[rank * B:(rank + 1) * B].sum() / (world * B)
    rel = lambda a, b: ((a.float() - b).abs().max() / (b.abs().max() + 1e-9)).item()  # noqa: E731
    cases.append({"B": B, "D": D, "rep": "negatives",
                  "loss_err": abs(loss.item() - share.item()) / max(1e-3, abs(share.item())),
                  "dq_err": rel(q.grad, Q.grad[rank * B:(rank + 1) * B]),
                  "dk_err": max(rel(d.grad, Kd.grad[rank * B:(rank + 1) * B]),
                                rel(n.grad, Kn.grad[rank * Bn:(rank + 1) * Bn]))})
    if rank == 0:
        with open(out_path, "w") as fh:
            json.dump({"cases": cases}, fh)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
