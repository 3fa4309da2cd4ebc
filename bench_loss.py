"""Distributed contrastive-loss micro-benchmark (forward + backward) at N GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench_loss.py [--sizes 1024,4096,8192] [--dims 768,1024,4096] [--iters 10]

Per rank: query and passage embeddings [B_local, D] bf16, N(0,1) then L2-normalised; global
similarity of the local queries against all ranks' passages / 0.02, row logsumexp, cross-entropy on
the diagonal targets, full backward with passage gradients returned to their owners.

Arms (each timed with CUDA events after warm-up, max over ranks; an L2-sized buffer is rewritten
between iterations):
  fused      lset_b200.dist.xrank_loss (peer pull fused into the tcgen05 similarity GEMM, dK
             reduce-scatter fused into the GEMM epilogue)
  nccl       NCCL all-gather / reduce-scatter around the same single-GPU streaming kernels
  ref_triton the reference's gather_with_grad + Triton fused_dense_loss (full global matrix per rank)
  ref_cuda   the reference's gather_with_grad + its CUDA fused_dense_loss_sm100
  ref_eager  the reference's gather_with_grad + infonce_loss (matmul + cross_entropy)
Reference arms run from baseline/_ref when importable; one JSON line per (B_local, D) on rank 0.
The roofline time of the fused path is max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s)
with FLOPs = 4 GEMMs of 2·B·(W·B)·D and NVLink bytes = inbound passages + outbound fp32 dK.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)  # rewrites a buffer larger than L2
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
    ap.add_argument("--sizes", default="1024,4096,8192")
    ap.add_argument("--dims", default="768,1024,4096")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-reference", action="store_true")
    args = ap.parse_args()
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())

    from lset_b200.dist.gather import gather_for_local_rows
    from lset_b200.dist.xrank_loss import cross_rank_infonce
    from lset_b200.ops import _native as nv
    from lset_b200.ops.loss import fused_infonce
    from lset_b200.utils.tracing import NVLINK_GBS_PER_DIRECTION, load_peaks

    # The reference's CUDA loss extension is compiled on first use (torch's JIT extension loader)
    # and looks for the CuTe headers under ~/workspace/cutlass/include. The image carries them
    # inside the flashinfer package instead: hand that directory to nvcc through its environment
    # hook, which leaves the reference's own build code untouched.
    import importlib.util

    spec = importlib.util.find_spec("flashinfer")
    cute = os.path.join(os.path.dirname(spec.origin), "data", "cutlass", "include") if spec else ""
    if os.path.isdir(cute):
        os.environ["NVCC_APPEND_FLAGS"] = (os.environ.get("NVCC_APPEND_FLAGS", "") + f" -I{cute}").strip()
    build_log = []

    class _Capture(__import__("logging").Handler):
        def emit(self, record):
            build_log.append(record.getMessage())

    __import__("logging").getLogger("lset.kernels.experimental.loss_sm100").addHandler(_Capture())
    dist.barrier()
    ref = {}
    if not args.no_reference and os.path.isdir(os.path.join(REPO, "baseline", "_ref", "lset")):
        sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
        try:
            from lset.distributed.gather import gather_with_grad
            from lset.kernels.loss import fused_dense_loss
            from lset.losses.infonce import infonce_loss as ref_infonce

            ref = {"gather": gather_with_grad, "triton": fused_dense_loss, "eager": ref_infonce}
            try:
                from lset.kernels.experimental import loss_sm100 as ref_sm100

                # build (or load from the JIT cache) now, rank by rank, and keep the reason if the
                # build fails: the wrapper itself only logs a warning and then fails on first use
                for r in range(world):
                    if r == rank and ref_sm100._load_sm100_extension() is None:
                        ref["cuda_err"] = ("build failed: " + " | ".join(build_log))[:400]
                    dist.barrier()
                if "cuda_err" not in ref:
                    ref["cuda"] = ref_sm100.fused_dense_loss_sm100
            except Exception as exc:  # pragma: no cover
                ref["cuda_err"] = repr(exc)[:200]
        except Exception as exc:  # pragma: no cover
            ref = {"err": repr(exc)[:200]}
    peaks = load_peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)  # 256 MB

    for B in [int(x) for x in args.sizes.split(",")]:
        for D in [int(x) for x in args.dims.split(",")]:
            torch.manual_seed(rank)
            q = F.normalize(torch.randn(B, D, device=dev), dim=-1).to(torch.bfloat16).requires_grad_()
            d = F.normalize(torch.randn(B, D, device=dev), dim=-1).to(torch.bfloat16).requires_grad_()

            def run_fused():
                q.grad = d.grad = None
                cross_rank_infonce(q, d, 0.02).backward()

            def run_nccl():
                q.grad = d.grad = None
                docs = gather_for_local_rows(d)
                (fused_infonce(q, docs, 0.02, rank * B) / world).backward()

            out = {"B_local": B, "D": D, "n_gpus": world, "dtype": "bf16", "iters": args.iters,
                   "fused_ms": timed(run_fused, args.iters, flush),
                   "nccl_ms": timed(run_nccl, args.iters, flush)}
            nv.check_status()
            flops = 4 * 2.0 * B * (world * B) * D
            link = (world - 1) * B * D * (2 + 4)
            t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), link / (NVLINK_GBS_PER_DIRECTION * 1e9))
            out["roofline_ms"] = 1e3 * t_roof
            out["fused_fraction_of_roofline"] = 1e3 * t_roof / out["fused_ms"]
            out["peaks"] = peaks.get("source")
            if "gather" in ref:
                N = world * B
                labels = None

                def make_ref(kind):
                    def run():
                        q.grad = d.grad = None
                        qa, da = ref["gather"](q), ref["gather"](d)
                        if kind == "eager":
                            ref["eager"](qa, da, 0.02).backward()
                        else:
                            ref[kind](qa, da, labels, 1.0 / 0.02).backward()
                    return run

                try:
                    if N * N <= 2 ** 31:
                        labels = torch.eye(N, dtype=torch.int8, device=dev)
                        out["ref_triton_ms"] = timed(make_ref("triton"), max(2, args.iters // 2), flush)
                        if "cuda" in ref:
                            try:
                                out["ref_cuda_ms"] = timed(make_ref("cuda"), max(2, args.iters // 2), flush)
                            except Exception as exc:
                                out["ref_cuda_ms"] = f"failed: {exc!r}"[:160]
                        else:
                            out["ref_cuda_ms"] = "unavailable: " + ref.get("cuda_err", "")
                        labels = None
                    else:
                        out["ref_triton_ms"] = "skipped: int8 label matrix over 2 GiB"
                    if N * N * 4 <= 24 * 2 ** 30:
                        out["ref_eager_ms"] = timed(make_ref("eager"), max(2, args.iters // 2), flush)
                except Exception as exc:  # pragma: no cover
                    out["ref_error"] = repr(exc)[:200]
            elif ref:
                out["ref_error"] = ref.get("err")
            if rank == 0:
                print(json.dumps(out), flush=True)
            del q, d
            torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
