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


def _extra_bytes(fn, q, k):
    """Peak memory of forward + backward beyond what was allocated before and the two gradient
    tensors that remain afterwards."""
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    fn().backward()
    torch.cuda.synchronize()
    grads = sum(t.grad.numel() * t.grad.element_size() for t in (q, k))
    return torch.cuda.max_memory_allocated() - base - grads


def test_no_score_matrix_in_any_precision():
    """The backward walks the passages in column panels: the bf16 probability gradient exists for
    one panel (capped at 64 MB, here an eighth of the score matrix) at a time, next to the fp32
    accumulator of dQ."""
    M, N, D = 8192, 32768, 256
    q, k = _emb(M, D, 4).requires_grad_(), _emb(N, D, 5).requires_grad_()
    extra = _extra_bytes(lambda: fused_infonce(q, k, 0.02), q, k)
    assert extra < M * N * 2 // 8 + M * D * 4 + (8 << 20), extra
    # and the panelled backward still matches the oracle
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    torch.nn.functional.cross_entropy(qr @ kr.t() / 0.02, torch.arange(M, device="cuda")).backward()
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad)):
        assert (a.float() - b).abs().max() < 3e-2 * (b.abs().max() + 1e-6)


def _eager_label_loss(q, k, labels, T, scores=None):
    """fp32 oracle: the formulas of the label-matrix loss written out with plain torch ops."""
    sim = q @ k.t() / T
    valid = labels >= 0
    lse = torch.logsumexp(sim.masked_fill(~valid, float("-inf")), dim=1)
    if scores is None:
        pos = (labels == 1).float()
        n = pos.sum(1)
        keep = (n > 0) & valid.any(1)
        per_q = lse - (sim * pos).sum(1) / n.clamp(min=1)
    else:
        t = scores.masked_fill(~valid, 0.0)
        ts = t.sum(1)
        keep = (ts > 0) & valid.any(1)
        per_q = lse - (t / ts.clamp(min=1e-12).unsqueeze(1) * sim).sum(1)
    return per_q[keep].mean()


@pytest.mark.parametrize("Q,K,D", [(64, 200, 256), (300, 1000, 1024), (128, 4096, 768), (40, 72, 128)])
@pytest.mark.parametrize("soft", [False, True])
def test_fused_label_loss_matches_eager(Q, K, D, soft):
    from lset_b200.ops.loss import fused_label_loss

    q, k = _emb(Q, D, 6).requires_grad_(), _emb(K, D, 7).requires_grad_()
    g = torch.Generator(device="cuda").manual_seed(Q + K)
    r = torch.rand(Q, K, device="cuda", generator=g)
    labels = torch.zeros(Q, K, device="cuda")
    labels[r < 0.02] = 1.0           # several positives per row
    labels[r > 0.9] = -1.0           # ignored columns
    labels[1] = 0.0                  # a query without positives is skipped
    labels[2] = -1.0                 # a query without any valid column too
    scores = torch.rand(Q, K, device="cuda", generator=g) * 4 if soft else None
    if soft:
        scores[3] = 0.0              # zero score sum: skipped
    loss = fused_label_loss(q, k, labels, 0.05, scores)
    loss.backward()
    nv.check_status()
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    ref = _eager_label_loss(qr, kr, labels, 0.05, scores)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
    for a, b, name in ((q.grad, qr.grad, "dq"), (k.grad, kr.grad, "dk")):
        err = (a.float() - b).abs().max().item()
        assert err < 3e-2 * (b.abs().max().item() + 1e-6), (name, err, b.abs().max().item())
    for row in ((2, 3) if soft else (1, 2)):   # the skipped queries get no gradient
        assert q.grad[row].abs().max().item() == 0.0


def test_label_loss_dispatches_to_streaming_kernels():
    from lset_b200.losses.contrastive import contrastive_loss

    Q, K = 2048, 4096
    q, k = _emb(Q, 256, 8).requires_grad_(), _emb(K, 256, 9).requires_grad_()
    labels = torch.zeros(Q, K, device="cuda")
    labels[torch.arange(Q), torch.arange(Q)] = 1.0
    before = nv.launches()
    extra = _extra_bytes(lambda: contrastive_loss(q, k, labels, 0.02), q, k)
    assert nv.launches() > before
    # int8 labels and masks derived from the label matrix ([Q, K] bytes each) and one column panel
    # of the bf16 probability gradient, but no score-sized fp32 or bf16 temporary (the eager
    # formulation holds at least three fp32 ones)
    assert extra < 6 * Q * K + Q * K * 2 + Q * 256 * 4 + (4 << 20), extra


def _eager_dense_loss(q, k, labels, scale, loss_type):
    """fp32 oracle of the three fused loss types, written from their definitions."""
    s = q @ k.t() * scale
    lab = labels.float()
    pos, neg, valid = lab > 0, lab == 0, lab >= 0
    if loss_type == "multi":
        neg_lse = torch.logsumexp(s.masked_fill(~neg, float("-inf")), dim=1, keepdim=True)
        per = F.softplus(neg_lse - s) * pos
        n_pos = pos.sum(1)
        keep = (n_pos > 0) & neg.any(1)
        per_q = per.sum(1) / n_pos.clamp(min=1)
        return per_q[keep].sum() / keep.sum().clamp(min=1)
    lse = torch.logsumexp(s.masked_fill(~valid, float("-inf")), dim=1)
    l = lab.clamp(min=0)
    lsum = l.sum(1)
    keep = lsum > 0
    if loss_type == "soft":
        per_q = lse - (l / lsum.clamp(min=1e-9).unsqueeze(1) * s).sum(1)
    else:
        per_q = lsum * lse - (l * s).sum(1)
    return per_q[keep].sum() / keep.sum().clamp(min=1)


@pytest.fixture
def small_panels(monkeypatch):
    """Makes the backward of the streaming losses walk several column panels at test sizes."""
    from lset_b200.ops import loss as loss_ops

    monkeypatch.setattr(loss_ops, "PANEL_BYTES", 256 * 1024)
    monkeypatch.setattr(loss_ops, "PANEL_MIN_COLS", 256)


def test_panelled_backward_of_infonce_and_label_losses(small_panels):
    """Several panels, a ragged last one, a target offset: same gradients as one panel."""
    from lset_b200.losses.contrastive import contrastive_loss
    from lset_b200.ops import loss as loss_ops

    M, N, D = 520, 1800, 256
    assert loss_ops.panel_cols(M, N) == 256
    q, k = _emb(M, D, 20).requires_grad_(), _emb(N, D, 21).requires_grad_()
    fused_infonce(q, k, 0.05, target_offset=700).backward()
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    F.cross_entropy(qr @ kr.t() / 0.05, torch.arange(M, device="cuda") + 700).backward()
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad)):
        assert (a.float() - b).abs().max() < 3e-2 * (b.abs().max() + 1e-6)
    labels = torch.zeros(M, N, device="cuda")
    labels[torch.arange(M), torch.arange(M) + 1000] = 1.0
    labels[:, 300:320] = -1
    q.grad = k.grad = None
    contrastive_loss(q, k, labels, 0.05).backward()
    qr.grad = kr.grad = None
    _eager_label_loss(qr, kr, labels, 0.05).backward()
    nv.check_status()
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad)):
        assert (a.float() - b).abs().max() < 3e-2 * (b.abs().max() + 1e-6)


@pytest.mark.parametrize("loss_type", ["multi", "soft", "cross"])
def test_fused_dense_loss_types_in_panels(small_panels, loss_type):
    test_fused_dense_loss_types(loss_type, 512, 2048, 1024, False)


@pytest.mark.parametrize("loss_type", ["multi", "soft", "cross"])
@pytest.mark.parametrize("Q,K,D,give_idx", [(96, 300, 256, True), (512, 2048, 1024, False)])
def test_fused_dense_loss_types(loss_type, Q, K, D, give_idx):
    from lset_b200.ops.loss import fused_dense_loss

    q, k = _emb(Q, D, 10).requires_grad_(), _emb(K, D, 11).requires_grad_()
    g = torch.Generator(device="cuda").manual_seed(3 * Q + K)
    r = torch.rand(Q, K, device="cuda", generator=g)
    labels = torch.zeros(Q, K, device="cuda", dtype=torch.int8)
    labels[r < 0.02] = 1
    if loss_type != "multi":
        labels[r < 0.01] = 3          # soft label values
    labels[r > 0.9] = -1
    labels[4] = 0                     # no positive: skipped
    labels[5] = torch.where(labels[5] == 0, torch.full_like(labels[5], -1), labels[5])  # no negative
    idx = (labels > 0).nonzero(as_tuple=True) if give_idx else (None, None)
    loss = fused_dense_loss(q, k, labels, 20.0, loss_type, pos_qi=idx[0], pos_di=idx[1])
    loss.backward()
    nv.check_status()
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    ref = _eager_dense_loss(qr, kr, labels, 20.0, loss_type)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
    for a, b, name in ((q.grad, qr.grad, "dq"), (k.grad, kr.grad, "dk")):
        err = (a.float() - b).abs().max().item()
        assert err < 3e-2 * (b.abs().max().item() + 1e-6), (name, err, b.abs().max().item())
    assert q.grad[4].abs().max().item() == 0.0


def test_fused_label_loss_reads_missing_teacher_scores_as_zero_targets():
    """Score matrices from the collator hold -inf for documents of other samples: the streaming
    kernels must treat them as targets of zero (in-batch negatives), with finite loss and
    gradients equal to the eager soft-label cross-entropy on the zero-filled scores."""
    from lset_b200.ops.loss import fused_label_loss

    Q, per, D = 96, 4, 512
    K = Q * per
    q, k = _emb(Q, D, 16).requires_grad_(), _emb(K, D, 17).requires_grad_()
    labels = torch.zeros(Q, K, device="cuda")
    scores = torch.full((Q, K), float("-inf"), device="cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    vals = torch.rand(Q, per, device="cuda", generator=g) * 3 + 0.1
    for j in range(per):
        cols = torch.arange(Q, device="cuda") * per + j
        scores[torch.arange(Q, device="cuda"), cols] = vals[:, j]
    labels[torch.arange(Q, device="cuda"), torch.arange(Q, device="cuda") * per] = 1.0
    loss = fused_label_loss(q, k, labels, 0.05, scores)
    loss.backward()
    nv.check_status()
    assert torch.isfinite(loss) and torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all()
    qr, kr = q.detach().float().requires_grad_(), k.detach().float().requires_grad_()
    ref = _eager_label_loss(qr, kr, labels, 0.05, torch.nan_to_num(scores, neginf=0.0))
    ref.backward()
    assert ref.item() > 0 and abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item()))
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad)):
        assert (a.float() - b).abs().max().item() < 3e-2 * (b.abs().max().item() + 1e-6)
