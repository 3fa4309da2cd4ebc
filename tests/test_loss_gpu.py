"""Streaming InfoNCE kernels against the fp32 eager loss: values, gradients, memory."""
import pytest
import torch
import torch.nn.functional as F

from lset_b200.ops import _native as nv
from lset_b200.ops.loss import fused_infonce, similarity

pytestmark = pytest.mark.gpu


def _emb(n, d, seed):
    torch.manual_seed(seed)
    return F.normalize(torch.randn(n, d, device="cuda"), dim=-1).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,D,off", [(64, 64, 1024, 0), (200, 456, 768, 0), (128, 1024, 256, 512),
                                       (1000, 3000, 1024, 1000), (8, 4096, 4096, 8)])
def test_fused_infonce_matches_eager(M, N, D, off):
    q, k = _emb(M, D, 0).requires_grad_(), _emb(N, D, 1).requires_grad_()
    loss = fused_infonce(q, k, 0.02, off)
    loss.backward()
    nv.check_status()
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    ref = F.cross_entropy(qr @ kr.t() / 0.02, torch.arange(M, device="cuda") + off)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
    for a, b, name in ((q.grad, qr.grad, "dq"), (k.grad, kr.grad, "dk")):
        err = (a.float() - b).abs().max().item()
        assert err < 3e-2 * (b.abs().max().item() + 1e-6), (name, err, b.abs().max().item())


def test_similarity_grads():
    q, k = _emb(40, 256, 2).requires_grad_(), _emb(72, 256, 3).requires_grad_()
    s = similarity(q, k)
    g = torch.randn_like(s)
    s.backward(g)
    ref_dq = g @ k.detach().float()
    assert (q.grad.float() - ref_dq).abs().max() < 3e-2 * ref_dq.abs().max()


def test_no_score_matrix_in_fp32():
    M, N, D = 2048, 4096, 1024
    q, k = _emb(M, D, 4).requires_grad_(), _emb(N, D, 5).requires_grad_()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    fused_infonce(q, k, 0.02).backward()
    torch.cuda.synchronize()
    assert torch.cuda.max_memory_allocated() - base < M * N * 4  # below one fp32 score matrix
