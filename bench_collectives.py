"""Micro-benchmark of the fused compute + collective kernels at N GPUs, each against its NCCL
composition and its roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench_collectives.py [--tokens 16384] [--iters 10]

Paths (one JSON line each on rank 0; ms = CUDA events, max over ranks, a 256 MB buffer rewritten
between iterations):
  ag_gemm      all-gather of token shards fused into the column-parallel GEMM (lb_gemm_bf16_ag)
               vs NCCL all_gather_into_tensor + the same GEMM kernel on local memory
  gemm_rs      row-parallel GEMM with the reduce-scatter fused into its epilogue
               (lb_gemm_bf16_scatter16: packed bf16x2 red.global.add to the owner; fp32 accumulators
               with LSET_B200_TP_RS_FP32=1) vs GEMM + NCCL reduce_scatter
  zero_step    sharded-optimizer step on a 256 Mi-parameter group: gradient reduce-scatter + average
               + ‖g‖² (lb_reduce_shard_f32) and AdamW + bf16 push all-gather (lb_adamw_push) vs NCCL
               reduce_scatter_tensor + the single-GPU AdamW kernel + all_gather_into_tensor
Shapes follow the Qwen3-4B tensor-parallel layer: hidden 2560, q/k/v 6144, FFN 9728 (x2 gate/up),
split over the N ranks.

Roofline time = max(FLOPs / measured cuBLAS bf16 peak, bytes that must cross NVLink per GPU and
direction / 770 GB/s, HBM bytes / measured copy bandwidth).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)
        flush.sum()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())

    from lset_b200.dist import tp_fused
    from lset_b200.dist.sharded import ParamStore, ShardedAdamW
    from lset_b200.ops import _native as nv
    from lset_b200.ops.gemm import matmul_abt
    from lset_b200.utils.tracing import NVLINK_GBS_PER_DIRECTION, load_peaks, roofline

    peaks = load_peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    st = tp_fused.SPState(dist.group.WORLD, dev)
    T = args.tokens // world * world
    rows = T // world
    H = 2560
    out = []

    def r(*shape):
        return (torch.randn(*shape, device=dev) * 0.05).to(torch.bfloat16)

    # ---------------------------------------------------------------- all-gather + GEMM
    for name, n_total in (("qkv", 6144), ("gate_up", 2 * 9728)):
        n_loc = n_total // world // 8 * 8
        x, w = r(rows, H), r(n_loc, H)

        def fused():
            tp_fused._ag_gemm(st, x, w, None, b_mn=False)

        def nccl():
            matmul_abt(st.all_gather_rows(x), w)

        ms_f, ms_n = timed(fused, args.iters, flush), timed(nccl, args.iters, flush)
        flops = 2.0 * T * n_loc * H
        link = 2.0 * (world - 1) * rows * H                       # inbound bf16 rows per GPU
        hbm = 2.0 * (T * H + n_loc * H + T * n_loc)
        out.append(dict(path="ag_gemm", layer=name, T=T, K=H, N_local=n_loc, fused_ms=ms_f,
                        nccl_ms=ms_n, **roofline(ms_f, flops, hbm, link, peaks)))

    # ---------------------------------------------------------------- GEMM + reduce-scatter
    for name, k_total in (("o_proj", 4096), ("down", 9728)):
        k_loc = k_total // world // 8 * 8
        x, w = r(T, k_loc), r(H, k_loc)

        def fused():
            tp_fused._gemm_rs(st, x, w, b_mn=False)

        def nccl():
            st.reduce_scatter_rows(matmul_abt(x, w))

        ms_f, ms_n = timed(fused, args.iters, flush), timed(nccl, args.iters, flush)
        flops = 2.0 * T * H * k_loc
        acc_bytes = 2.0 if st.rs_bf16 else 4.0
        link = acc_bytes * (world - 1) * rows * H                 # outbound partial rows
        hbm = 2.0 * (T * k_loc + H * k_loc) + acc_bytes * rows * H * 2
        out.append(dict(path="gemm_rs", layer=name, T=T, K_local=k_loc, N=H, fused_ms=ms_f,
                        nccl_ms=ms_n, **roofline(ms_f, flops, hbm, link, peaks)))
    nv.check_status(dev)

    # ---------------------------------------------------------------- sharded optimizer step
    n_par = 256 * 1024 * 1024
    for symm_on in (True, False):
        os.environ["LSET_B200_SYMM"] = "1" if symm_on else "0"
        lin = torch.nn.Linear(16384, n_par // 16384, bias=False)
        store = ParamStore(lin, layer_modules=[lin], dp_group=dist.group.WORLD,
                           compute_dtype=torch.bfloat16, device=dev)
        opt = ShardedAdamW(store, lr=1e-4, grad_clip=1.0)
        g = store.groups[0]

        def step():
            g.flat_grad.normal_(0.0, 1e-3)     # stands in for the backward pass (not a collective)
            g.reduced = False
            store.finish_backward()
            opt.step()
            store.wait_all_gathers()

        def grad_only():
            g.flat_grad.normal_(0.0, 1e-3)

        ms = timed(step, args.iters, flush) - timed(grad_only, args.iters, flush)
        shard = n_par // world
        link = max(4.0 * (world - 1) * shard, 2.0 * (world - 1) * shard)   # fp32 in, bf16 out
        hbm = 4.0 * n_par / world * world + shard * (4 * 3 * 2 + 2) + 2.0 * n_par
        key = "fused_ms" if symm_on else "nccl_ms"
        if symm_on:
            # With gradient clipping the update needs the global norm, i.e. the whole reduction,
            # first: the step is two dependent sweeps, each with its own binding resource.
            # Sweep 1 (reduce): fp32 shards of the W - 1 peers come in over NVLink; this GPU's
            # memory serves its own shard, the peers' reads of theirs, and the reduced write.
            # Sweep 2 (AdamW + push): fp32 gradient, two moments and the master read and written,
            # the bf16 shard written locally and into W - 1 peers, whose pushes land here.
            nvl = NVLINK_GBS_PER_DIRECTION * 1e9
            hbm_bw = peaks["hbm_gbs"] * 1e9
            p1 = max(4.0 * (world - 1) * shard / nvl, 4.0 * shard * (world + 1) / hbm_bw)
            p2 = max(2.0 * (world - 1) * shard / nvl, shard * (30.0 + 2.0 * (world - 1)) / hbm_bw)
            floor_ms = (p1 + p2) * 1e3
            out.append(dict(path="zero_step", params=n_par, symm=bool(store.use_symm), fused_ms=ms,
                            two_phase_floor_ms=floor_ms, fraction_of_two_phase_floor=floor_ms / ms,
                            **roofline(ms, 0.0, hbm, link, peaks)))
        else:
            out[-1][key] = ms
        del store, opt, lin, g
        torch.cuda.empty_cache()
    os.environ["LSET_B200_SYMM"] = "1"
    nv.check_status(dev)

    if rank == 0:
        for line in out:
            line["n_gpus"] = world
            print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
