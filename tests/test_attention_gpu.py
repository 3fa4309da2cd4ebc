"""Varlen attention kernels against the fp32 eager oracle (ragged sequences, GQA, both masks)."""
import pytest
import torch

from lset_b200.ops import _native as nv
from lset_b200.ops.attention import AttnPlan, attention_ref, varlen_attention

pytestmark = pytest.mark.gpu


def _make(lens, Hq, Hk, hd, fused=False, seed=0):
    torch.manual_seed(seed)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    if fused:
        qkv = torch.randn(T, Hq + 2 * Hk, hd, device="cuda").to(torch.bfloat16)
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hk], qkv[:, Hq + Hk:]
    else:
        q = torch.randn(T, Hq, hd, device="cuda").to(torch.bfloat16)
        k = torch.randn(T, Hk, hd, device="cuda").to(torch.bfloat16)
        v = torch.randn(T, Hk, hd, device="cuda").to(torch.bfloat16)
    return q, k, v, cu, AttnPlan(cu, max(lens), T)


CASES = [
    ([64], 2, 2, 128), ([128], 2, 1, 128), ([17, 200, 64, 333], 4, 2, 128),
    ([40, 512, 129, 1], 16, 8, 128), ([300, 77], 8, 2, 128), ([250, 31], 8, 1, 128),
    ([100, 260], 4, 4, 64), ([90, 130], 2, 1, 256),
]


@pytest.mark.parametrize("lens,Hq,Hk,hd", CASES)
@pytest.mark.parametrize("causal", [True, False])
def test_forward(lens, Hq, Hk, hd, causal):
    q, k, v, cu, plan = _make(lens, Hq, Hk, hd)
    o = varlen_attention(q, k, v, plan, causal)
    nv.check_status()
    ref = attention_ref(q.float(), k.float(), v.float(), cu, causal)
    err = (o.float() - ref).abs().max().item()
    assert err < 3e-2, err


def test_forward_fused_qkv_views():
    q, k, v, cu, plan = _make([70, 190, 33], 16, 8, 128, fused=True)
    o = varlen_attention(q, k, v, plan, True)
    nv.check_status()
    ref = attention_ref(q.float(), k.float(), v.float(), cu, True)
    assert (o.float() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("lens,Hq,Hk,hd", CASES)
@pytest.mark.parametrize("causal", [True, False])
def test_backward(lens, Hq, Hk, hd, causal):
    q, k, v, cu, plan = _make(lens, Hq, Hk, hd, seed=1)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    o = varlen_attention(q, k, v, plan, causal)
    g = torch.randn_like(o)
    o.backward(g)
    nv.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_ref(qr, kr, vr, cu, causal)
    ref.backward(g.float())
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        scale = b.abs().max().item() + 1e-6
        assert err / scale < 3e-2, (name, err, scale)


@pytest.mark.parametrize("left", [True, False])
def test_padded_plan(left):
    torch.manual_seed(3)
    B, S, Hq, Hk, hd = 3, 96, 4, 2, 128
    lens = [96, 40, 7]
    mask = torch.zeros(B, S, dtype=torch.long, device="cuda")
    for b, L in enumerate(lens):
        if left:
            mask[b, S - L:] = 1
        else:
            mask[b, :L] = 1
    plan = AttnPlan.from_mask(mask)
    q = torch.randn(B * S, Hq, hd, device="cuda").to(torch.bfloat16)
    k = torch.randn(B * S, Hk, hd, device="cuda").to(torch.bfloat16)
    v = torch.randn(B * S, Hk, hd, device="cuda").to(torch.bfloat16)
    o = varlen_attention(q, k, v, plan, True)
    nv.check_status()
    ref = attention_ref(q.float(), k.float(), v.float(), plan.seq_start, True, seq_end=plan.seq_end)
    assert (o.float() - ref).abs().max().item() < 3e-2


def test_stream_padded_past_the_last_sequence():
    """A packed stream padded to a fixed token budget: the tokens behind the last sequence belong
    to no sequence. Their output and gradient rows are cleared (no kernel writes them), and what
    they hold on input does not reach the rows of real tokens."""
    lens, pad = [70, 190, 33], 150
    Hq, Hk, hd = 8, 4, 128
    q, k, v, cu, plan = _make(lens, Hq, Hk, hd, seed=5)
    T = sum(lens)
    big = lambda h: (torch.randn(pad, h, hd, device="cuda") * 50).to(torch.bfloat16)  # noqa: E731
    qp, kp, vp = (torch.cat([t, big(t.shape[1])]).requires_grad_() for t in (q, k, v))
    plan_p = AttnPlan(cu, max(lens), T + pad)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    o = varlen_attention(q, k, v, plan, True)
    g = torch.randn_like(o)
    o.backward(g)
    # poison the allocator's free blocks so that "never written" shows up as garbage
    junk = torch.full((T + pad, Hq, hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    del junk
    op = varlen_attention(qp, kp, vp, plan_p, True)
    op.backward(torch.cat([g, torch.zeros(pad, Hq, hd, device="cuda", dtype=g.dtype)]))
    nv.check_status()
    assert torch.equal(op[:T], o) and not op[T:].any()
    for a, b in ((qp.grad, q.grad), (kp.grad, k.grad), (vp.grad, v.grad)):
        assert torch.equal(a[:T], b) and not a[T:].any()
