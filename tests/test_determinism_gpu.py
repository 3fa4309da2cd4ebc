"""Run-to-run determinism of the kernels whose results do not depend on the order of atomics:
the same inputs twice must give bitwise equal outputs. A data race inside a kernel (a missing
barrier, a shared-memory stage reused too early, a TMEM accumulator read before its commit) shows
up here as a difference between two runs long before it shows up as a numerical error.

Kernels that reduce with floating-point atomics by design (split-K weight gradients, embedding
backward, the cross-rank scatter of the loss) are excluded: their sums depend on arrival order.
"""
import pytest
import torch

from lset_b200.ops import _native as nv
from lset_b200.ops import activation as A
from lset_b200.ops import fp8 as f8
from lset_b200.ops import norm as N
from lset_b200.ops import rope as R
from lset_b200.ops.attention import AttnPlan, varlen_attention
from lset_b200.ops.gemm import matmul_abt

pytestmark = pytest.mark.gpu

REPEATS = 3


def _r(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _same(fn):
    """Call ``fn`` REPEATS times; every returned tensor must be bitwise equal across the calls."""
    first = None
    for _ in range(REPEATS):
        out = fn()
        out = out if isinstance(out, (tuple, list)) else (out,)
        out = [o.detach().clone() for o in out if o is not None]
        torch.cuda.synchronize()
        if first is None:
            first = out
        else:
            for i, (a, b) in enumerate(zip(first, out)):
                assert torch.equal(a, b), f"output {i} differs between runs"
    nv.check_status()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_forms(a_mn, b_mn):
    torch.manual_seed(0)
    M, N, K = 1504, 1032, 520   # MN-major operands need leading dimensions that are multiples of 8
    a = _r(K, M) if a_mn else _r(M, K)
    b = _r(K, N) if b_mn else _r(N, K)
    _same(lambda: matmul_abt(a, b, a_mn=a_mn, b_mn=b_mn))
    _same(lambda: matmul_abt(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32))


def test_fp8_cast_and_gemm():
    torch.manual_seed(1)
    x, w = _r(1500, 1024), _r(776, 1024)

    def cast():
        q, q_t = f8.quantize_fp8(x, f8.PER_TENSOR, want_t=True)
        _, c_t = f8.quantize_fp8(x, f8.PER_COL, e5m2=True, want=False, want_t=True)
        return q.data, q_t.data, q.inv_scale, c_t.data, c_t.inv_scale

    _same(cast)
    xq, _ = f8.quantize_fp8(x, f8.PER_ROW)
    wq, _ = f8.quantize_fp8(w, f8.PER_ROW)
    _same(lambda: f8.matmul_fp8(xq, wq))


@pytest.mark.parametrize("causal", [True, False])
def test_attention_forward_and_backward(causal):
    torch.manual_seed(2)
    lens = [40, 512, 129, 1, 300, 77]
    T, Hq, Hk, hd = sum(lens), 16, 8, 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    plan = AttnPlan(cu, max(lens), T)
    q, k, v = _r(T, Hq, hd), _r(T, Hk, hd), _r(T, Hk, hd)
    g = _r(T, Hq, hd)

    def run():
        qq, kk, vv = (t.detach().clone().requires_grad_() for t in (q, k, v))
        o = varlen_attention(qq, kk, vv, plan, causal)
        o.backward(g)
        return o, qq.grad, kk.grad, vv.grad

    _same(run)


def test_norms_rope_and_glu():
    torch.manual_seed(3)
    n, H = 1000, 1024
    x, res, w, g = _r(n, H), _r(n, H), _r(H, scale=0.5), _r(n, H)

    def norm():
        xx, rr = x.detach().clone().requires_grad_(), res.detach().clone().requires_grad_()
        y, nr = N.residual_rms_norm(rr, xx, w, 1e-6)
        torch.autograd.backward([y, nr], [g, g])
        return y, nr, xx.grad, rr.grad

    _same(norm)

    Hq, Hk, hd = 16, 8, 128
    qkv = _r(n, Hq + 2 * Hk, hd)
    qw, kw = _r(hd, scale=0.5), _r(hd, scale=0.5)
    pos = torch.randint(0, 700, (n,), device="cuda")
    cos, sin = R.rope_tables(hd, 1024, 1e6, "cuda")
    gq, gk = _r(n, Hq, hd), _r(n, Hk, hd)

    def rope():
        t = qkv.detach().clone().requires_grad_()
        qo, ko = R.qk_norm_rope(t[:, :Hq], t[:, Hq:Hq + Hk], qw, kw, cos, sin, pos)
        torch.autograd.backward([qo, ko], [gq, gk])
        return qo, ko, t.grad

    _same(rope)

    gu, gg = _r(n, 2 * 3072), _r(n, 3072)

    def glu():
        t = gu.detach().clone().requires_grad_()
        y = A.glu(t, "swiglu")
        y.backward(gg)
        return y, t.grad

    _same(glu)
