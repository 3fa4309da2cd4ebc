"""Single-kernel micro-benchmarks with roofline fractions (also the small cases that the ncu
captures under ``profiles/`` are taken from).

    python -m lset_b200.utils.kernel_bench gemm  --m 23040 --n 4096 --k 1024 [--form fprop|dgrad|wgrad]
                                                 [--ref torch]   (torch.matmul / cuBLAS alongside)
    python -m lset_b200.utils.kernel_bench fp8   --m 23040 --n 4096 --k 1024 [--what gemm|cast|linear]
    python -m lset_b200.utils.kernel_bench attn  --seqs 64 --len 320 --hq 16 --hk 8 --hd 128 [--bwd]
                                                 [--ref flash]   (flash_attn_varlen_func alongside)
    python -m lset_b200.utils.kernel_bench norm  --rows 23040 --h 1024 [--bwd]
    python -m lset_b200.utils.kernel_bench rope  --rows 23040 --hq 16 --hk 8 --hd 128 [--bwd]
    python -m lset_b200.utils.kernel_bench glu   --rows 23040 --i 3072 [--bwd]
    python -m lset_b200.utils.kernel_bench loss  --q 8192 --k 8192 --d 1024
    python -m lset_b200.utils.kernel_bench pool  --seqs 4096 --len 64 --h 1024 [--bwd]
    python -m lset_b200.utils.kernel_bench embed --rows 131072 --h 1024 [--bwd]
    python -m lset_b200.utils.kernel_bench adamw --n 268435456

Timing: CUDA events on the launching stream, 3 warm-up launches, a 256 MB buffer rewritten and then
read between timed launches (larger than the 126 MB L2; the read leaves no dirty lines whose
write-back would be charged to the timed kernel). One JSON line per run.
"""
from __future__ import annotations

import argparse
import json

import torch

from .tracing import roofline


def _time(fn, iters: int) -> float:
    flush = torch.zeros(64 * 1024 * 1024, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        for _ in range(4):   # also gives the host time to enqueue fn() behind the flush
            flush.add_(1.0)
        flush.sum()   # the read pass pushes the dirty lines of the write pass out of L2
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def _r(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def bench_gemm(a):
    from ..ops.gemm import matmul_abt

    M, N, K = a.m, a.n, a.k
    if a.form == "fprop":
        x, w = _r(M, K), _r(N, K)
        fn = lambda: matmul_abt(x, w, bn=a.bn)  # noqa: E731
    elif a.form == "dgrad":
        dy, w = _r(M, N), _r(N, K)
        fn = lambda: matmul_abt(dy, w, b_mn=True, bn=a.bn)  # noqa: E731  [M,K] = dy · w
    else:
        dy, x = _r(M, N), _r(M, K)
        out = torch.zeros(N, K, device="cuda")
        fn = lambda: matmul_abt(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True,  # noqa: E731
                                splits=a.splits)
    ms = _time(fn, a.iters)
    flops = 2.0 * M * N * K
    byt = 2.0 * (M * K + N * K + M * N)
    out = dict(kernel=f"gemm_{a.form}", M=M, N=N, K=K, ms=ms, **roofline(ms, flops, byt))
    if a.ref == "torch":
        # the library GEMM (cuBLAS through torch.matmul) on the same operands, same timing method
        if a.form == "fprop":
            ref = lambda: torch.matmul(x, w.t())  # noqa: E731
        elif a.form == "dgrad":
            ref = lambda: torch.matmul(dy, w)  # noqa: E731
        else:
            ref = lambda: torch.matmul(dy.t(), x)  # noqa: E731
        out["torch_matmul_ms"] = _time(ref, a.iters)
        out["torch_over_ours"] = out["torch_matmul_ms"] / ms
    return out


def bench_fp8(a):
    """8-bit GEMM alone (operands quantised beforehand), the cast of its activation operand, or
    quantise + GEMM as the fp8 linear layer runs them; the bf16 GEMM of the same shape alongside."""
    from ..ops import fp8 as f8
    from ..ops.gemm import matmul_abt

    M, N, K = a.m, a.n, a.k
    x, w = _r(M, K), _r(N, K)
    mode = f8.PER_ROW if a.rowwise else f8.PER_TENSOR
    xq, _ = f8.quantize_fp8(x, mode)
    wq, _ = f8.quantize_fp8(w, mode)
    flops = 2.0 * M * N * K
    if a.what == "gemm":
        fn = lambda: f8.matmul_fp8(xq, wq)  # noqa: E731
        byt = 1.0 * (M * K + N * K) + 2.0 * M * N
    elif a.what == "cast":
        fn = lambda: f8.quantize_fp8(x, mode, want_t=not a.rowwise)  # noqa: E731
        flops, byt = 0.0, (2.0 * 2 + (1.0 if a.rowwise else 2.0)) * M * K   # two reads of x
    else:
        def fn():
            q, _ = f8.quantize_fp8(x, mode)
            f8.matmul_fp8(q, wq)
        byt = (2.0 * 2 + 1.0 + 1.0) * M * K + 1.0 * N * K + 2.0 * M * N
    ms = _time(fn, a.iters)
    ms_bf16 = _time(lambda: matmul_abt(x, w), a.iters)
    return dict(kernel=f"fp8_{a.what}", rowwise=bool(a.rowwise), M=M, N=N, K=K, ms=ms,
                bf16_gemm_ms=ms_bf16, **roofline(ms, flops, byt))


def bench_attn(a):
    from ..ops.attention import AttnPlan, varlen_attention

    lens = [a.len] * a.seqs
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    plan = AttnPlan(cu, a.len, T)
    q, k, v = _r(T, a.hq, a.hd), _r(T, a.hk, a.hd), _r(T, a.hk, a.hd)
    pairs = a.seqs * (a.len * (a.len + 1) / 2 if a.causal else a.len * a.len)
    if a.bwd:
        q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
        o = varlen_attention(q, k, v, plan, a.causal)
        g = _r(T, a.hq, a.hd)
        fn = lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True)  # noqa: E731
        flops = 10.0 * pairs * a.hq * a.hd
    else:
        fn = lambda: varlen_attention(q, k, v, plan, a.causal)  # noqa: E731
        flops = 4.0 * pairs * a.hq * a.hd
    ms = _time(fn, a.iters)
    out = dict(kernel="attn_bwd" if a.bwd else "attn_fwd", seqs=a.seqs, len=a.len, Hq=a.hq, Hk=a.hk,
               hd=a.hd, causal=a.causal, ms=ms, **roofline(ms, flops, 0.0))
    if a.ref == "flash":
        # flash-attn's varlen kernels (what the reference calls) on the same tensors
        try:
            from flash_attn import flash_attn_varlen_func
        except Exception as exc:  # pragma: no cover - optional package
            out["flash_attn"] = f"unavailable: {exc!r}"[:120]
            return out
        qf, kf, vf = (t.detach().clone().requires_grad_(a.bwd) for t in (q, k, v))
        run = lambda: flash_attn_varlen_func(qf, kf, vf, cu, cu, a.len, a.len,  # noqa: E731
                                             causal=bool(a.causal))
        if a.bwd:
            of = run()
            gf = _r(T, a.hq, a.hd)
            ref = lambda: torch.autograd.grad(of, (qf, kf, vf), gf, retain_graph=True)  # noqa: E731
        else:
            ref = lambda: run()  # noqa: E731
        out["flash_attn_ms"] = _time(ref, a.iters)
        out["flash_over_ours"] = out["flash_attn_ms"] / ms
    return out


def bench_norm(a):
    from ..ops.norm import residual_rms_norm

    r, x, w = _r(a.rows, a.h), _r(a.rows, a.h), _r(a.h)
    if a.bwd:
        x.requires_grad_(); r.requires_grad_(); w.requires_grad_()
        y, nr = residual_rms_norm(r, x, w)
        g1, g2 = _r(a.rows, a.h), _r(a.rows, a.h)
        fn = lambda: torch.autograd.grad((y, nr), (x, w), (g1, g2), retain_graph=True)  # noqa: E731
        byt = 2.0 * a.rows * a.h * 4
    else:
        fn = lambda: residual_rms_norm(r, x, w)  # noqa: E731
        byt = 2.0 * a.rows * a.h * 4
    ms = _time(fn, a.iters)
    return dict(kernel="residual_rms_norm_" + ("bwd" if a.bwd else "fwd"), rows=a.rows, H=a.h, ms=ms,
                **roofline(ms, 0.0, byt))


def bench_rope(a):
    from ..ops.rope import qk_norm_rope, rope_tables

    qkv = _r(a.rows, a.hq + 2 * a.hk, a.hd)
    q, k = qkv[:, :a.hq], qkv[:, a.hq:a.hq + a.hk]
    qw, kw = _r(a.hd), _r(a.hd)
    cos, sin = rope_tables(a.hd, 1024, 1e6, "cuda")
    pos = torch.randint(0, 512, (a.rows,), device="cuda")
    n = a.rows * (a.hq + a.hk) * a.hd
    if a.bwd:
        qq, kk = q.detach().requires_grad_(), k.detach().requires_grad_()
        qo, ko = qk_norm_rope(qq, kk, qw, kw, cos, sin, pos)
        g1, g2 = torch.randn_like(qo), torch.randn_like(ko)
        fn = lambda: torch.autograd.grad((qo, ko), (qq, kk), (g1, g2), retain_graph=True)  # noqa: E731
        byt = 2.0 * n * 3
    else:
        fn = lambda: qk_norm_rope(q, k, qw, kw, cos, sin, pos)  # noqa: E731
        byt = 2.0 * n * 2
    ms = _time(fn, a.iters)
    return dict(kernel="qk_norm_rope_" + ("bwd" if a.bwd else "fwd"), rows=a.rows, ms=ms,
                **roofline(ms, 0.0, byt))


def bench_glu(a):
    from ..ops.activation import glu

    gu = _r(a.rows, 2 * a.i)
    if a.bwd:
        gu.requires_grad_()
        y = glu(gu)
        g = _r(a.rows, a.i)
        fn = lambda: torch.autograd.grad(y, gu, g, retain_graph=True)  # noqa: E731
        byt = 2.0 * a.rows * a.i * 5
    else:
        fn = lambda: glu(gu)  # noqa: E731
        byt = 2.0 * a.rows * a.i * 3
    ms = _time(fn, a.iters)
    return dict(kernel="swiglu_" + ("bwd" if a.bwd else "fwd"), rows=a.rows, I=a.i, ms=ms,
                **roofline(ms, 0.0, byt))


def bench_loss(a):
    import torch.nn.functional as F

    from ..ops.loss import fused_infonce

    q = F.normalize(torch.randn(a.q, a.d, device="cuda"), dim=-1).to(torch.bfloat16).requires_grad_()
    k = F.normalize(torch.randn(a.k, a.d, device="cuda"), dim=-1).to(torch.bfloat16).requires_grad_()

    def fn():
        q.grad = k.grad = None
        fused_infonce(q, k, 0.02).backward()

    ms = _time(fn, a.iters)
    return dict(kernel="infonce_fwd_bwd", Q=a.q, K=a.k, D=a.d, ms=ms,
                **roofline(ms, 8.0 * a.q * a.k * a.d, 0.0))


def bench_pool(a):
    from ..ops.pooling import packed_pool

    T = a.seqs * a.len
    h = _r(T, a.h)
    cu = torch.arange(a.seqs + 1, device="cuda", dtype=torch.int32) * a.len
    if a.bwd:
        h.requires_grad_()
        y = packed_pool(h, cu, "mean", True)
        g = _r(a.seqs, a.h)
        fn = lambda: torch.autograd.grad(y, h, g, retain_graph=True)  # noqa: E731
        byt = 2.0 * T * a.h
    else:
        fn = lambda: packed_pool(h, cu, "mean", True)  # noqa: E731
        byt = 2.0 * T * a.h
    ms = _time(fn, a.iters)
    return dict(kernel="segment_mean_l2norm_" + ("bwd" if a.bwd else "fwd"), seqs=a.seqs, len=a.len,
                H=a.h, ms=ms, **roofline(ms, 0.0, byt))


def bench_embed(a):
    from ..ops.embedding import embedding

    table = _r(151936, a.h)
    ids = torch.randint(0, 151936, (a.rows,), device="cuda")
    if a.bwd:
        table.requires_grad_()
        y = embedding(ids, table)
        g = _r(a.rows, a.h)
        fn = lambda: torch.autograd.grad(y, table, g, retain_graph=True)  # noqa: E731
        byt = a.rows * a.h * (2.0 + 8.0)      # read bf16 grads, fp32 read-modify-write of the rows
    else:
        fn = lambda: embedding(ids, table)  # noqa: E731
        byt = a.rows * a.h * 4.0
    ms = _time(fn, a.iters)
    return dict(kernel="embedding_" + ("bwd" if a.bwd else "fwd"), rows=a.rows, H=a.h, ms=ms,
                **roofline(ms, 0.0, byt))


def bench_adamw(a):
    from ..dist.sharded import ParamStore, ShardedAdamW

    lin = torch.nn.Linear(16384, a.n // 16384, bias=False)
    store = ParamStore(lin, layer_modules=[lin], compute_dtype=torch.bfloat16,
                       device=torch.device("cuda"))
    opt = ShardedAdamW(store, lr=1e-4, grad_clip=1.0)
    store.groups[0].flat_grad.normal_(0.0, 1e-3)

    def fn():
        store.sumsq.zero_()
        opt.step()

    ms = _time(fn, a.iters)
    # grad read twice (norm, update), master + two moments read and written, bf16 copy written
    byt = a.n * (4.0 * 2 + 4.0 * 6 + 2.0)
    return dict(kernel="sumsq+clip+adamw", n=a.n, ms=ms, **roofline(ms, 0.0, byt))


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="which", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=23040); g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=1024); g.add_argument("--form", default="fprop")
    g.add_argument("--bn", type=int, default=0); g.add_argument("--splits", type=int, default=0)
    g.add_argument("--ref", choices=["none", "torch"], default="none")
    f = sub.add_parser("fp8")
    f.add_argument("--m", type=int, default=23040); f.add_argument("--n", type=int, default=4096)
    f.add_argument("--k", type=int, default=1024); f.add_argument("--what", default="gemm")
    f.add_argument("--rowwise", action="store_true")
    t = sub.add_parser("attn")
    t.add_argument("--seqs", type=int, default=64); t.add_argument("--len", type=int, default=320)
    t.add_argument("--hq", type=int, default=16); t.add_argument("--hk", type=int, default=8)
    t.add_argument("--hd", type=int, default=128); t.add_argument("--bwd", action="store_true")
    t.add_argument("--bidirectional", dest="causal", action="store_false")
    t.add_argument("--ref", choices=["none", "flash"], default="none")
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=23040); n.add_argument("--h", type=int, default=1024)
    n.add_argument("--bwd", action="store_true")
    r = sub.add_parser("rope")
    r.add_argument("--rows", type=int, default=23040); r.add_argument("--hq", type=int, default=16)
    r.add_argument("--hk", type=int, default=8); r.add_argument("--hd", type=int, default=128)
    r.add_argument("--bwd", action="store_true")
    u = sub.add_parser("glu")
    u.add_argument("--rows", type=int, default=23040); u.add_argument("--i", type=int, default=3072)
    u.add_argument("--bwd", action="store_true")
    l = sub.add_parser("loss")
    l.add_argument("--q", type=int, default=8192); l.add_argument("--k", type=int, default=8192)
    l.add_argument("--d", type=int, default=1024)
    po = sub.add_parser("pool")
    po.add_argument("--seqs", type=int, default=4096); po.add_argument("--len", type=int, default=64)
    po.add_argument("--h", type=int, default=1024); po.add_argument("--bwd", action="store_true")
    em = sub.add_parser("embed")
    em.add_argument("--rows", type=int, default=131072); em.add_argument("--h", type=int, default=1024)
    em.add_argument("--bwd", action="store_true")
    ad = sub.add_parser("adamw")
    ad.add_argument("--n", type=int, default=268435456)
    for p in (g, f, t, n, r, u, l, po, em, ad):
        p.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    from ..ops import _native as nv

    out = {"gemm": bench_gemm, "fp8": bench_fp8, "attn": bench_attn, "norm": bench_norm, "rope": bench_rope,
           "glu": bench_glu, "loss": bench_loss, "pool": bench_pool, "embed": bench_embed,
           "adamw": bench_adamw}[a.which](a)
    nv.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
