"""8-bit float GEMM on the tensor cores (tcgen05 ``kind::f8f6f4``) and the dynamic-scaling casts
that feed it.

``quantize_fp8`` turns a bf16 matrix into e4m3 / e5m2 bytes with one scale per tensor, per row or
per column (``lb_fp8_amax`` + ``lb_fp8_cast``) and can emit the transposed copy in the same pass;
``matmul_fp8`` multiplies two K-major quantised operands and dequantises in the epilogue
(``lb_gemm_fp8``: row factor of A times row factor of B, fp32 accumulation in tensor memory).
On the CPU both run the same arithmetic in plain PyTorch (the oracle of the GPU tests).

Native counterpart of the torchao float8 kernels the reference switches on with ``fp8.enabled``
(lset/train/quantization/fp8.py:11-45).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _native as nv

E4M3_MAX, E5M2_MAX = 448.0, 57344.0
AMAX_FLOOR = 1e-12
PER_TENSOR, PER_ROW, PER_COL = 0, 1, 2


@dataclass
class Fp8Tensor:
    """Quantised matrix: ``data`` ``[rows, ld]`` bytes (the first ``cols`` of each row are valid),
    ``inv_scale`` fp32 with one element (per tensor) or ``rows`` elements, ``e5m2`` format flag."""
    data: torch.Tensor
    cols: int
    inv_scale: torch.Tensor
    e5m2: bool

    @property
    def rows(self) -> int:
        return self.data.shape[0]

    def dequantize(self) -> torch.Tensor:
        dt = torch.float8_e5m2 if self.e5m2 else torch.float8_e4m3fn
        f = self.data[:, :self.cols].view(dt).float()
        s = self.inv_scale if self.inv_scale.numel() == 1 else self.inv_scale[:, None]
        return f * s


def _round16(n: int) -> int:
    return (n + 15) // 16 * 16


def _quantize_eager(x, mode, e5m2, want, want_t):
    fmax = E5M2_MAX if e5m2 else E4M3_MAX
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    xf = x.float()
    if mode == PER_TENSOR:
        amax = xf.abs().amax().reshape(1)
    elif mode == PER_ROW:
        amax = xf.abs().amax(dim=1)
    else:
        amax = xf.abs().amax(dim=0)
    amax = amax.clamp(min=AMAX_FLOOR)
    scale = torch.full_like(amax, fmax) / amax     # a true division, as the kernel does
    if mode == PER_ROW:
        q = xf * scale[:, None]
    elif mode == PER_COL:
        q = xf * scale[None, :]
    else:
        q = xf * scale
    q = q.clamp(-fmax, fmax).to(dt).view(torch.uint8)
    inv = (amax / fmax).float()
    R, C = x.shape
    out = out_t = None
    if want:
        if mode == PER_COL:
            raise ValueError("per-column scales belong to the transposed output")
        out = Fp8Tensor(q.contiguous(), C, inv, e5m2)
    if want_t:
        if mode == PER_ROW:
            raise ValueError("per-row scales belong to the row-major output")
        ld = _round16(R)
        buf = torch.zeros(C, ld, dtype=torch.uint8, device=x.device)
        buf[:, :R] = q.t()
        out_t = Fp8Tensor(buf, R, inv, e5m2)
    return out, out_t


def quantize_fp8(x: torch.Tensor, mode: int = PER_TENSOR, *, e5m2: bool = False,
                 want: bool = True, want_t: bool = False):
    """Quantise a 2-D bf16 matrix ``x [R, C]`` (C a multiple of 8).

    ``mode``: PER_TENSOR (one scale), PER_ROW (one per row of ``x``: the row-major output is then
    scaled along its contraction dim) or PER_COL (one per column of ``x`` = per row of the
    transposed output). Returns ``(q, q_t)``: ``q`` is ``x`` row-major, ``q_t`` is ``xᵀ``
    (``[C, R]``, rows padded to a multiple of 16 bytes); either is None when not requested.
    """
    if x.dim() != 2:
        raise ValueError("quantize_fp8 takes a 2-D matrix")
    R, C = x.shape
    if not nv.use_native(x):
        return _quantize_eager(x, mode, e5m2, want, want_t)
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    if x.stride(1) != 1 or x.stride(0) % 8:
        x = x.contiguous()
    if C % 8:
        raise ValueError("quantize_fp8 needs a multiple of 8 columns")
    if mode == PER_COL and want:
        raise ValueError("per-column scales belong to the transposed output")
    if mode == PER_ROW and want_t:
        raise ValueError("per-row scales belong to the row-major output")
    dev = x.device
    n_scale = 1 if mode == PER_TENSOR else (R if mode == PER_ROW else C)
    amax = torch.empty(n_scale, dtype=torch.int32, device=dev)
    inv = torch.empty(n_scale, dtype=torch.float32, device=dev)
    out = torch.empty(R, C, dtype=torch.uint8, device=dev) if want else None
    ldt = _round16(R)
    out_t = torch.empty(C, ldt, dtype=torch.uint8, device=dev) if want_t else None
    lib = nv.load()
    stream = nv.c_void_p(nv.stream_ptr())
    rc = lib.lb_fp8_amax(nv.c_void_p(x.data_ptr()), nv.c_int(R), nv.c_int(C),
                         nv.c_ll(x.stride(0)), nv.c_int(mode), nv.c_void_p(amax.data_ptr()), stream)
    if rc != 0:
        nv.check_rc(rc, f"lb_fp8_amax(R={R},C={C})")
    rc = lib.lb_fp8_cast(nv.c_void_p(x.data_ptr()), nv.c_int(R), nv.c_int(C),
                         nv.c_ll(x.stride(0)), nv.c_int(mode), nv.c_void_p(amax.data_ptr()),
                         nv.c_int(int(e5m2)), nv.c_void_p(nv.ptr(out)), nv.c_ll(C),
                         nv.c_void_p(nv.ptr(out_t)), nv.c_ll(ldt), nv.c_void_p(inv.data_ptr()),
                         stream)
    if rc != 0:
        nv.check_rc(rc, f"lb_fp8_cast(R={R},C={C})")
    nv.count_launch(2)
    q = Fp8Tensor(out, C, inv, e5m2) if want else None
    q_t = Fp8Tensor(out_t, R, inv, e5m2) if want_t else None
    return q, q_t


def matmul_fp8(a: Fp8Tensor, b: Fp8Tensor, *, out: Optional[torch.Tensor] = None,
               out_dtype=torch.bfloat16, accumulate: bool = False, bias=None, splits: int = 1):
    """``C[M, N] = dequant(A) · dequant(B)ᵀ`` for K-major quantised ``a [M, K]`` and ``b [N, K]``.

    fp32 accumulation; the scale factors are applied to the accumulator. ``out`` fp32 with
    ``accumulate=True`` adds into it (weight gradients); ``splits`` as in ``matmul_abt``.
    """
    M, N, K = a.rows, b.rows, a.cols
    if b.cols != K:
        raise ValueError(f"contraction mismatch: {K} vs {b.cols}")
    if out is not None:
        out_dtype = out.dtype
    if not nv.use_native(a.data, b.data):
        c = a.dequantize() @ b.dequantize().t()
        if bias is not None:
            c = c + bias.float()
        if out is not None:
            if accumulate:
                out.add_(c.to(out.dtype))
            else:
                out.copy_(c)
            return out
        return c.to(out_dtype)
    if N % 8:
        raise ValueError("matmul_fp8 needs N to be a multiple of 8")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("output must be bf16 or fp32")
    if out_dtype != torch.float32:
        splits = 1
    auto = splits == 0      # the launcher picks the split (it may reduce into ``out``)
    if out is None:
        alloc = torch.zeros if (accumulate or splits != 1) else torch.empty
        out = alloc(M, N, dtype=out_dtype, device=a.data.device)
    elif splits != 1 and not accumulate:
        out.zero_()
    if M == 0 or N == 0:
        return out
    if bias is not None and bias.dtype != torch.bfloat16:
        bias = bias.to(torch.bfloat16)
    rc = nv.load().lb_gemm_fp8(
        nv.c_void_p(a.data.data_ptr()), nv.c_void_p(b.data.data_ptr()), nv.c_void_p(out.data_ptr()),
        nv.c_int(M), nv.c_int(N), nv.c_int(K),
        nv.c_ll(a.data.stride(0)), nv.c_ll(b.data.stride(0)), nv.c_ll(out.stride(0)),
        nv.c_int(int(a.e5m2)), nv.c_int(int(b.e5m2)),
        nv.c_void_p(a.inv_scale.data_ptr()), nv.c_int(int(a.inv_scale.numel() > 1)),
        nv.c_void_p(b.inv_scale.data_ptr()), nv.c_int(int(b.inv_scale.numel() > 1)),
        nv.c_int(int(out_dtype == torch.float32)), nv.c_int(int(accumulate or splits > 1 or auto)),
        nv.c_void_p(nv.ptr(bias)), nv.c_int(splits), nv.c_int(0),
        nv.c_void_p(nv.status_word(a.data.device).data_ptr()), nv.c_void_p(nv.stream_ptr()))
    if rc != 0:
        nv.check_rc(rc, f"lb_gemm_fp8(M={M},N={N},K={K})")
    nv.count_launch()
    return out
