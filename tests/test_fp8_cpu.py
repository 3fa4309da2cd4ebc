"""FP8 training on the CPU: the eager quantise → multiply → rescale path of ``ops/fp8.py`` and the
``Float8Linear`` recipes (cf. lset/train/quantization/fp8.py:11-45)."""
import pytest
import torch
import torch.nn as nn

from lset_b200.ops import fp8 as f8
from lset_b200.train.quantization.fp8 import RECIPES, Float8Linear, apply_fp8_training


def test_quantize_layouts_and_scales():
    torch.manual_seed(0)
    x = torch.randn(37, 24) * 3.0
    q, q_t = f8.quantize_fp8(x, f8.PER_TENSOR, want_t=True)
    assert q.data.shape == (37, 24) and q_t.data.shape == (24, 48) and q_t.cols == 37
    assert q.inv_scale.numel() == 1
    assert torch.equal(q_t.data[:, :37], q.data.t())
    assert int(q_t.data[:, 37:].max()) == 0
    # the largest magnitude maps onto the largest finite e4m3 value
    assert float(q.dequantize().abs().max()) == pytest.approx(float(x.abs().max()), rel=1e-6)
    assert torch.allclose(q.dequantize(), x, rtol=0.07, atol=float(x.abs().max()) * 2 ** -9)

    qr, _ = f8.quantize_fp8(x, f8.PER_ROW)
    assert qr.inv_scale.shape == (37,)
    assert torch.allclose(qr.dequantize().abs().amax(1), x.abs().amax(1), rtol=1e-6)
    _, qc = f8.quantize_fp8(x, f8.PER_COL, e5m2=True, want=False, want_t=True)
    assert qc.inv_scale.shape == (24,) and qc.e5m2
    assert torch.allclose(qc.dequantize().abs().amax(1), x.abs().amax(0), rtol=1e-6)
    with pytest.raises(ValueError):
        f8.quantize_fp8(x, f8.PER_COL)
    with pytest.raises(ValueError):
        f8.quantize_fp8(x, f8.PER_ROW, want_t=True)


def test_matmul_fp8_matches_dequantised_product():
    torch.manual_seed(1)
    a, b = torch.randn(19, 32), torch.randn(40, 32)
    aq, _ = f8.quantize_fp8(a, f8.PER_ROW)
    bq, _ = f8.quantize_fp8(b, f8.PER_TENSOR)
    c = f8.matmul_fp8(aq, bq, out_dtype=torch.float32)
    assert torch.allclose(c, aq.dequantize() @ bq.dequantize().t(), atol=1e-5)
    acc = torch.ones(19, 40)
    f8.matmul_fp8(aq, bq, out=acc, accumulate=True)
    assert torch.allclose(acc, c + 1.0, atol=1e-5)


@pytest.mark.parametrize("recipe", RECIPES)
def test_float8_linear_tracks_full_precision(recipe):
    torch.manual_seed(2)
    lin = nn.Linear(64, 48)
    ref = nn.Linear(64, 48)
    ref.load_state_dict(lin.state_dict())
    apply_fp8_training(lin, recipe)
    assert isinstance(lin, Float8Linear)
    x = torch.randn(3, 11, 64, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    y, yr = lin(x), ref(xr)
    assert y.dtype == torch.float32 and y.shape == yr.shape
    g = torch.randn_like(yr)
    y.backward(g)
    yr.backward(g)

    def rel(u, v):
        return float((u - v).abs().max() / v.abs().max())

    assert rel(y.detach(), yr.detach()) < 0.08
    assert rel(x.grad, xr.grad) < 0.12          # e5m2 output gradients: 2 mantissa bits
    assert rel(lin.weight.grad, ref.weight.grad) < (1e-5 if recipe.endswith("gw_hp") else 0.12)
    assert torch.allclose(lin.bias.grad, ref.bias.grad, atol=1e-5)


def test_ineligible_layers_are_left_alone():
    m = nn.Sequential(nn.Linear(30, 16), nn.Linear(16, 32))
    apply_fp8_training(m, "tensorwise")
    assert type(m[0]) is nn.Linear and isinstance(m[1], Float8Linear)
    with pytest.raises(ValueError):
        apply_fp8_training(m, "blockwise")
