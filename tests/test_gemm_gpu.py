"""tcgen05 GEMM against a plain PyTorch fp32 reference, all operand layouts and ragged shapes."""
import pytest
import torch

from lset_b200.ops import _native as nv
from lset_b200.ops.gemm import linear, matmul_abt

pytestmark = pytest.mark.gpu


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def _check(c, ref, tol=2e-2):
    nv.check_status()
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale:.4g}"


SHAPES = [(128, 256, 64), (256, 512, 128), (300, 264, 200), (1000, 1024, 1024), (4096, 3072, 1024),
          (77, 128, 72), (513, 1032, 520)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bn", [0, 128, 256])
def test_nt(M, N, K, bn):
    a, b = _rand(M, K), _rand(N, K)
    c = matmul_abt(a, b, bn=bn)
    _check(c, a.float() @ b.float().t())


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_nn_b_mn_major(M, N, K):
    a, b = _rand(M, K), _rand(K, N)
    c = matmul_abt(a, b, b_mn=True)
    _check(c, a.float() @ b.float())


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("splits", [1, 3])
def test_tn_both_mn_major_fp32(M, N, K, splits):
    a, b = _rand(K, M if M % 8 == 0 else M + (8 - M % 8)), _rand(K, N)
    Mp = a.shape[1]
    c = matmul_abt(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32, splits=splits)
    assert c.shape == (Mp, N)
    _check(c, a.float().t() @ b.float(), tol=5e-3)


def test_a_mn_b_k():
    a, b = _rand(192, 256), _rand(320, 192)
    c = matmul_abt(a, b, a_mn=True)
    _check(c, a.float().t() @ b.float().t())


def test_accumulate_and_bias():
    a, b = _rand(256, 128), _rand(256, 128)
    bias = _rand(256)
    c = matmul_abt(a, b, bias=bias)
    _check(c, a.float() @ b.float().t() + bias.float())
    out = torch.ones(256, 256, device="cuda")
    matmul_abt(a, b, out=out, accumulate=True)
    _check(out, a.float() @ b.float().t() + 1.0, tol=5e-3)


def test_deterministic():
    a, b = _rand(2048, 1024), _rand(1024, 1024)
    c1 = matmul_abt(a, b)
    c2 = matmul_abt(a, b)
    assert torch.equal(c1, c2)


def test_linear_autograd():
    x = _rand(4, 130, 256).requires_grad_()
    w = _rand(512, 256).requires_grad_()
    bias = _rand(512).requires_grad_()
    y = linear(x, w, bias)
    g = _rand(4, 130, 512)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    _check(y, yr.detach())
    _check(x.grad, xr.grad)
    _check(w.grad, wr.grad)
    _check(bias.grad, br.grad)
