"""tcgen05 GEMM against a plain PyTorch fp32 reference, all operand layouts and ragged shapes."""
import pytest
import torch

from lset_b200.ops import _native as nv
from lset_b200.ops.gemm import linear, matmul_abt

pytestmark = pytest.mark.gpu


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


@pytest.fixture(autouse=True, params=["pair", "single"])
def gemm_kernel(request):
    """Every test runs twice: with the CTA-pair kernel (256 x 256 tiles on 2-CTA clusters, the
    default for plain products of at least one such tile) and with the one-CTA kernel only."""
    lib = nv.load()
    before = lib.lb_gemm_use_2cta(-1)
    lib.lb_gemm_use_2cta(1 if request.param == "pair" else 0)
    yield request.param
    lib.lb_gemm_use_2cta(before)


def _check(c, ref, tol=2e-2):
    """Error relative to the magnitude of the 64 x 64 block it falls in (floored at a twentieth of
    the global maximum), so that a wrong or missing tile cannot hide behind large values elsewhere."""
    nv.check_status()
    c = c.float()
    if ref.dim() == 1:
        c, ref = c[None], ref[None]
    c, ref = c.reshape(-1, c.shape[-1]), ref.reshape(-1, ref.shape[-1])
    err = (c - ref).abs()
    M, N = ref.shape
    Mp, Np = -(-M // 64) * 64, -(-N // 64) * 64
    pad = lambda t: torch.nn.functional.pad(t, (0, Np - N, 0, Mp - M))  # noqa: E731
    blk = lambda t: pad(t).view(Mp // 64, 64, Np // 64, 64).amax(dim=(1, 3))  # noqa: E731
    scale = blk(ref.abs()).clamp_min(0.05 * ref.abs().max().item() + 1e-6)
    worst = (blk(err) / scale).max().item()
    assert worst < tol, f"worst block-relative error {worst:.4g}"


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


@pytest.mark.parametrize("M,N,K,K2", [(300, 512, 256, 16), (1000, 4096, 1024, 16), (64, 128, 128, 8),
                                      (513, 1024, 2560, 64)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_matmul_ext_second_operand_pair(M, N, K, K2, b_mn):
    """C = A·op(B) + A2·op(B2) in one accumulator pass (the LoRA forward / input-gradient form)."""
    from lset_b200.ops.gemm import matmul_ext

    torch.manual_seed(0)
    r = lambda *s: (torch.randn(*s, device="cuda") * 0.3).to(torch.bfloat16)  # noqa: E731
    a, a2 = r(M, K), r(M, K2)
    b, b2 = (r(K, N), r(K2, N)) if b_mn else (r(N, K), r(N, K2))
    bias = None if b_mn else r(N)
    c = matmul_ext(a, b, a2, b2, b_mn=b_mn, bias=bias)
    nv.check_status()
    bf, b2f = (b.float(), b2.float()) if b_mn else (b.float().t(), b2.float().t())
    ref = a.float() @ bf + a2.float() @ b2f + (bias.float() if bias is not None else 0.0)
    err = (c.float() - ref).abs().max().item()
    assert err < 2e-2 * ref.abs().max().item(), (err, ref.abs().max().item())


def test_lora_linear_matches_three_products():
    from lset_b200.models.layers import Linear
    from lset_b200.train.lora import LoRALinear

    torch.manual_seed(1)
    base = Linear(512, 768, bias=False, device="cuda", dtype=torch.bfloat16)
    lora = LoRALinear(base, r=16, alpha=32.0).to("cuda")
    torch.nn.init.normal_(lora.lora_B.weight, std=0.05)      # away from the zero initialisation
    x = (torch.randn(3, 100, 512, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    g = (torch.randn(3, 100, 768, device="cuda") * 0.5).to(torch.bfloat16)
    assert lora._fusable(x)
    y = lora(x)
    y.backward(g)
    nv.check_status()
    got = (y.detach(), x.grad, lora.lora_A.weight.grad, lora.lora_B.weight.grad)
    xr = x.detach().float().requires_grad_()
    W, A, B = (t.detach().float().requires_grad_() for t in
               (base.weight, lora.lora_A.weight, lora.lora_B.weight))
    yr = xr @ W.t() + (xr @ A.t()) @ B.t() * lora.scale
    yr.backward(g.float())
    for a, b, name in zip(got, (yr.detach(), xr.grad, A.grad, B.grad), ("y", "dx", "dA", "dB")):
        err = (a.float() - b).abs().max().item()
        assert err < 3e-2 * b.abs().max().item(), (name, err, b.abs().max().item())
    assert base.weight.grad is None


@pytest.mark.parametrize("T,I,K", [(300, 512, 256), (1000, 3072, 1024), (77, 200, 128), (2048, 9728, 2560)])
@pytest.mark.parametrize("kind", ["swiglu", "geglu"])
def test_linear_glu_epilogue(T, I, K, kind):
    """Gate/up projection with the activation in the GEMM epilogue against the two-kernel path
    (same rounding points) and against fp32 PyTorch, values and gradients."""
    from lset_b200.ops.activation import glu
    from lset_b200.ops.gemm import linear_glu

    torch.manual_seed(2)
    x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(2 * I, K, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    g = (torch.randn(T, I, device="cuda") * 0.5).to(torch.bfloat16)
    h = linear_glu(x, w, kind)
    h.backward(g)
    nv.check_status()
    got = (h.detach(), x.grad.clone(), w.grad.clone())
    x.grad = w.grad = None
    h2 = glu(linear(x, w), kind)
    h2.backward(g)
    two = (h2.detach(), x.grad, w.grad)
    # same rounding points as the two-kernel path: equal up to a last-bit difference of the activation
    assert (got[0].float() - two[0].float()).abs().max() <= 1e-2 * two[0].float().abs().max()
    for a, b, name in zip(got[1:], two[1:], ("dx", "dw")):
        assert (a.float() - b.float()).abs().max() <= 1e-2 * b.float().abs().max(), name
    xr, wr = x.detach().float(), w.detach().float()
    gu = xr @ wr.t()
    act = torch.nn.functional.silu(gu[:, :I]) if kind == "swiglu" else \
        torch.nn.functional.gelu(gu[:, :I], approximate="tanh")
    ref = act * gu[:, I:]
    assert (got[0].float() - ref).abs().max() < 3e-2 * ref.abs().max()
