"""8-bit tensor-core GEMM (tcgen05 kind::f8f6f4) and its cast kernels against plain PyTorch fp32:
the quantised bytes against the eager cast, the product against the fp32 product of the
dequantised operands, and the fp8 linear layer against the same layer run on the CPU path."""
import pytest
import torch
import torch.nn as nn

from lset_b200.ops import _native as nv
from lset_b200.ops import fp8 as f8
from lset_b200.train.quantization.fp8 import RECIPES, apply_fp8_training

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=0.5):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _rel(c, ref):
    return float((c.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-9))


def _to_cpu(q):
    return f8.Fp8Tensor(q.data.cpu(), q.cols, q.inv_scale.cpu(), q.e5m2)


@pytest.mark.parametrize("R,C", [(64, 64), (300, 264), (77, 1024), (1000, 72), (5, 8)])
@pytest.mark.parametrize("mode", [f8.PER_TENSOR, f8.PER_ROW, f8.PER_COL])
@pytest.mark.parametrize("e5m2", [False, True])
def test_cast_matches_eager(R, C, mode, e5m2):
    x = _rand(R, C, scale=2.0)
    x[0, :] = 0  # an all-zero row
    want, want_t = mode != f8.PER_COL, mode != f8.PER_ROW
    q, q_t = f8.quantize_fp8(x, mode, e5m2=e5m2, want=want, want_t=want_t)
    qe, qe_t = f8.quantize_fp8(x.cpu(), mode, e5m2=e5m2, want=want, want_t=want_t)
    nv.check_status()
    for got, exp in ((q, qe), (q_t, qe_t)):
        if exp is None:
            assert got is None
            continue
        assert got.data.shape == exp.data.shape and got.cols == exp.cols
        assert torch.allclose(got.inv_scale.cpu(), exp.inv_scale, rtol=1e-6)
        same = (got.data.cpu() == exp.data).float().mean().item()
        assert same >= 0.9999, f"only {same:.5f} of the bytes agree"
        assert torch.allclose(_to_cpu(got).dequantize(), exp.dequantize(),
                              rtol=0.13 if not e5m2 else 0.26, atol=1e-6)
        if got is q_t:
            assert int(got.data[:, got.cols:].max().item() if got.data.shape[1] > got.cols else 0) == 0


GEMM_SHAPES = [(128, 256, 128), (256, 512, 256), (300, 264, 208), (1000, 1024, 1024),
               (4096, 3072, 1024), (77, 128, 80), (513, 1032, 528), (23040, 1024, 3072)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("modes", [(f8.PER_TENSOR, f8.PER_TENSOR), (f8.PER_ROW, f8.PER_ROW),
                                   (f8.PER_ROW, f8.PER_TENSOR)])
def test_gemm_against_fp32_of_dequantised(M, N, K, modes):
    a, b = _rand(M, K), _rand(N, K)
    aq, _ = f8.quantize_fp8(a, modes[0])
    bq, _ = f8.quantize_fp8(b, modes[1])
    c = f8.matmul_fp8(aq, bq)
    nv.check_status()
    ref = aq.dequantize() @ bq.dequantize().t()
    assert c.dtype == torch.bfloat16 and c.shape == (M, N)
    assert _rel(c, ref) < 1e-2                      # bf16 rounding of the output only
    assert _rel(c, a.float() @ b.float().t()) < 0.1  # and fp8-close to the unquantised product


def test_gemm_formats_bias_fp32_accumulate_and_splits():
    M, N, K = 520, 384, 2000 // 16 * 16
    a, b = _rand(M, K), _rand(N, K)
    bias = _rand(N)
    aq, _ = f8.quantize_fp8(a, f8.PER_ROW, e5m2=True)          # e5m2 x e4m3 (gradient products)
    bq, _ = f8.quantize_fp8(b, f8.PER_ROW)
    ref = aq.dequantize() @ bq.dequantize().t()
    c = f8.matmul_fp8(aq, bq, bias=bias)
    assert _rel(c, ref + bias.float()) < 1e-2
    bq5, _ = f8.quantize_fp8(b, f8.PER_TENSOR, e5m2=True)      # e5m2 on the B side
    assert _rel(f8.matmul_fp8(aq, bq5, out_dtype=torch.float32),
                aq.dequantize() @ bq5.dequantize().t()) < 1e-4
    out = torch.ones(M, N, device="cuda")
    f8.matmul_fp8(aq, bq, out=out, accumulate=True, splits=4)
    nv.check_status()
    assert _rel(out, ref + 1.0) < 1e-4


def test_weight_gradient_form_from_transposed_copies():
    T, N, K = 3000, 256, 512                       # dW[N, K] = dyᵀ · x, contraction over the tokens
    dy, x = _rand(T, N), _rand(T, K)
    _, dyq_t = f8.quantize_fp8(dy, f8.PER_COL, e5m2=True, want=False, want_t=True)
    _, xq_t = f8.quantize_fp8(x, f8.PER_COL, want=False, want_t=True)
    dw = f8.matmul_fp8(dyq_t, xq_t, out_dtype=torch.float32, splits=3)
    nv.check_status()
    assert _rel(dw, dyq_t.dequantize() @ xq_t.dequantize().t()) < 1e-4
    assert _rel(dw, dy.float().t() @ x.float()) < 0.1


@pytest.mark.parametrize("recipe", RECIPES)
def test_float8_linear_matches_cpu_path(recipe):
    torch.manual_seed(3)
    lin = nn.Linear(256, 384).to(torch.bfloat16)
    ref = nn.Linear(256, 384).to(torch.bfloat16)
    ref.load_state_dict(lin.state_dict())
    lin = apply_fp8_training(lin.cuda(), recipe)
    apply_fp8_training(ref, recipe)
    x = (torch.randn(4, 75, 256) * 0.5).to(torch.bfloat16)
    g = (torch.randn(4, 75, 384) * 0.5).to(torch.bfloat16)
    xg = x.cuda().requires_grad_()
    xc = x.clone().requires_grad_()
    before = nv.launches()
    y = lin(xg)
    y.backward(g.cuda())
    assert nv.launches() > before                  # the native kernels ran, not a fallback
    yr = ref(xc)
    yr.backward(g)
    nv.check_status()
    assert _rel(y.detach().cpu(), yr.detach()) < 2e-2
    assert _rel(xg.grad.cpu(), xc.grad) < 3e-2
    assert _rel(lin.weight.grad.cpu(), ref.weight.grad) < 3e-2
    assert _rel(lin.bias.grad.cpu(), ref.bias.grad) < 2e-2
    # and against the full-precision layer: fp8-close
    full = nn.Linear(256, 384).to(torch.bfloat16)
    full.load_state_dict(ref.state_dict())
    assert _rel(y.detach().cpu(), full(x).detach()) < 0.1


@pytest.mark.parametrize("recipe", ["tensorwise", "rowwise"])
def test_engine_trains_with_fp8_linears(recipe):
    """A small Qwen3 embedder through the engine with fp8 linear layers: first-step loss and
    gradient direction stay close to the bf16 run, and the loss goes down."""
    from lset_b200.models import Qwen3Config
    from lset_b200.train.data.collator import PackedCollator
    from lset_b200.train.data.dataset import SyntheticPairDataset
    from lset_b200.train.engine import TrainingEngine
    from lset_b200.train.quantization.fp8 import Float8Linear

    cfg = Qwen3Config(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    ds = SyntheticPairDataset(64, 2048, (8, 24), (40, 200), seed=3)
    batch = PackedCollator()([ds[i] for i in range(8)])

    def engine(**kw):
        torch.manual_seed(0)
        return TrainingEngine("qwen3", None, None, batch_size=8, lr=1e-3, packed=True,
                              model_config=cfg, log_interval=0, scheduler_type="constant",
                              fused_projections=True, device="cuda", **kw)

    ref, eng = engine(), engine(fp8=True, fp8_recipe=recipe)
    assert sum(isinstance(m, Float8Linear) for m in eng.model.modules()) >= 8
    l_ref = float(ref.forward_backward(batch, True))
    l_fp8 = float(eng.forward_backward(batch, True))
    nv.check_status()
    assert abs(l_fp8 - l_ref) < 0.1 * max(1.0, abs(l_ref)), (l_fp8, l_ref)
    flat = lambda e: torch.cat([g.flat_grad.float().cpu() for g in e.store.groups])  # noqa: E731
    cos = torch.nn.functional.cosine_similarity(flat(eng), flat(ref), dim=0).item()
    assert cos > 0.9, cos
    eng.optimizer_step()
    losses = [float(eng.train_step(batch)) for _ in range(8)]
    assert losses[-1] < losses[0], losses
