"""Worker of the fused tensor-parallel test (one process per GPU, launched by torch.distributed.run).

Checks, against plain fp32 PyTorch on the gathered operands:
  * ``ag_linear``  (all-gather fused into the GEMM) forward and both gradients,
  * ``linear_rs``  (reduce-scatter fused into the GEMM epilogue) forward and both gradients,
  * a small Qwen3 decoder under sequence-parallel tensor parallelism against the unsharded model.
Writes the maximal relative errors as JSON (rank 0).
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))


def main():
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())
    from lset_b200.dist import tp_fused
    from lset_b200.ops import _native as nv

    st = tp_fused.SPState(dist.group.WORLD, dev)
    res = {"fused": bool(st.fused), "cases": []}

    def gather(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return parts

    for rows, K, N in ((192, 256, 512), (300, 1024, 384), (64, 128, 128), (86, 256, 256),
                       (86, 128, 256), (45, 256, 512)):
        for it in range(3):  # three uses: both halves of the double buffers and a reuse
            torch.manual_seed(100 * it + rank)
            x = (torch.randn(rows, K, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
            torch.manual_seed(7 + it)  # the same full weight on every rank, sliced per rank
            w_col_full = (torch.randn(world * N, K, device=dev) * 0.05).to(torch.bfloat16)
            w_col = w_col_full[rank * N:(rank + 1) * N].clone().requires_grad_()
            bias = (torch.randn(N, device=dev) * 0.1).to(torch.bfloat16).requires_grad_()
            # ---- all-gather + GEMM
            y = tp_fused.ag_linear(x, w_col, bias, st)
            gy = (torch.randn(world * rows, N, device=dev) * 0.5).to(torch.bfloat16)
            y.backward(gy)
            x_all = torch.cat(gather(x.detach()))
            y_ref = x_all.float() @ w_col.detach().float().t() + bias.detach().float()
            dx_part = gy.float() @ w_col.detach().float()          # [T, K] partial of this rank
            dist.all_reduce(dx_part)
            dx_ref = dx_part[rank * rows:(rank + 1) * rows]
            dw_ref = gy.float().t() @ x_all.float()
            case = {"op": "ag_linear", "rows": rows, "K": K, "N": N, "it": it,
                    "y": rel(y, y_ref), "dx": rel(x.grad, dx_ref), "dw": rel(w_col.grad, dw_ref),
                    "db": rel(bias.grad, gy.float().sum(0))}
            res["cases"].append(case)
            # ---- GEMM + reduce-scatter: x2 [T, K] holds this rank's K slice of the features
            x2 = (torch.randn(world * rows, K, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
            w_row = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
            y2 = tp_fused.linear_rs(x2, w_row, None, st)
            gy2 = (torch.randn(rows, N, device=dev) * 0.5).to(torch.bfloat16)
            y2.backward(gy2)
            part = x2.detach().float() @ w_row.detach().float().t()
            dist.all_reduce(part)
            y2_ref = part[rank * rows:(rank + 1) * rows]
            gy2_all = torch.cat(gather(gy2))
            dx2_ref = gy2_all.float() @ w_row.detach().float()
            dw2_ref = gy2_all.float().t() @ x2.detach().float()
            res["cases"].append({"op": "linear_rs", "rows": rows, "K": K, "N": N, "it": it,
                                 "y": rel(y2, y2_ref), "dx": rel(x2.grad, dx2_ref),
                                 "dw": rel(w_row.grad, dw2_ref)})
    nv.check_status()

    # ---- whole model: sequence-parallel Qwen3 vs the unsharded model
    from lset_b200.dist.tp import apply_tp
    from lset_b200.models import Qwen3Config, Qwen3Decoder
    from lset_b200.models.layers import init_normal_
    from lset_b200.models.parallel_plan import decoder_tp_plan

    # whole heads per rank at every world size
    cfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=max(4, 2 * world), num_key_value_heads=max(2, world),
                      head_dim=64)
    torch.manual_seed(0)
    ref = Qwen3Decoder(cfg, fused_projections=True)
    init_normal_(ref, 0.05)
    full = {k: v.clone() for k, v in ref.state_dict().items()}
    ref = ref.to(dev, torch.bfloat16)
    lens = [37, 64, 50, 21]
    T = sum(lens)
    ids = torch.arange(T, device=dev) % 512
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    pos = torch.cat([torch.arange(n, device=dev) for n in lens])

    # A fixed random projection as the loss: sum(h²) after the final RMSNorm is (almost) constant,
    # its gradient is rounding noise and would compare nothing.
    torch.manual_seed(11)
    proj = torch.randn(T, cfg.hidden_size, device=dev) / T

    def run(model):
        h = model.forward_packed(ids, pos, cu, max(lens))["hidden_states"]
        (h.float() * proj).sum().backward()
        return h.detach()

    def sharded_model(fused):
        mm = Qwen3Decoder(cfg, fused_projections=True)
        mm.load_state_dict(full)
        apply_tp(mm, dist.group.WORLD, decoder_tp_plan(cfg, fused_projections=True,
                                                       use_sequence_parallel=True))
        mm = mm.to(dev, torch.bfloat16)
        mm._sp.bind(dev)
        if not fused:
            mm._sp.fused = False   # plain all-gather / reduce-scatter around local GEMMs
        return mm

    outs = [run(ref)]
    m_plain = sharded_model(False)
    h_plain = run(m_plain)
    m = sharded_model(True)
    outs.append(run(m))
    res["plain_vs_fused"] = {
        "hidden": rel(outs[1], h_plain),
        "worst_grad": max(rel(a.grad, b.grad) for a, b in zip(m.parameters(), m_plain.parameters())
                          if a.grad is not None)}
    # every parameter gradient of the sharded models against the matching slice of the reference
    from lset_b200.dist.tp import _section_sizes, _shard_rows

    ref_params = dict(ref.named_parameters())

    def grad_errors(model):
        grads = {}
        for name, p in model.named_parameters():
            g_ref = ref_params[name].grad
            g_tp = p.grad
            if g_tp is None or g_ref is None:
                continue
            if getattr(p, "_tp_sharded", False):
                mod_name = name.rsplit(".", 1)[0]
                mod = ref.get_submodule(mod_name)
                owner = ref.get_submodule(mod_name.rsplit(".", 1)[0])
                if g_tp.shape[0] != g_ref.shape[0]:      # column-parallel: rows sharded by section
                    g_ref = _shard_rows(g_ref, _section_sizes(mod_name, mod, owner), rank, world)
                else:                                     # row-parallel: input features sharded
                    per = g_ref.shape[1] // world
                    g_ref = g_ref[:, rank * per:(rank + 1) * per]
            elif getattr(p, "_tp_partial_grad", False):
                g_tp = g_tp.float().clone()
                dist.all_reduce(g_tp)                    # the sharding runtime sums these over the group
            grads[name] = rel(g_tp, g_ref)
        return grads

    grads, grads_plain = grad_errors(m), grad_errors(m_plain)
    res["model"] = {"hidden": rel(outs[1], outs[0]), "grads": grads, "grads_plain": grads_plain,
                    "worst_grad": max(grads.values()), "worst_grad_plain": max(grads_plain.values()),
                    "sp_fused": bool(m._sp.fused)}
    nv.check_status()
    dist.barrier()
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(res, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
