"""Losses: InfoNCE, label-matrix contrastive (multi-positive, soft labels, ignore), matryoshka,
LogitScale, and the bi-encoder task."""
import math

import pytest
import torch
import torch.nn.functional as F

from lset_b200.losses import (LogitScale, contrastive_loss, fused_contrastive_loss, infonce_loss,
                              matryoshka_loss)


def _emb(n, d, seed):
    torch.manual_seed(seed)
    return F.normalize(torch.randn(n, d), dim=-1)


def test_infonce_matches_cross_entropy_and_extra_negatives():
    q, d = _emb(6, 16, 0), _emb(9, 16, 1)
    ref = F.cross_entropy(q @ d.t() / 0.05, torch.arange(6))
    assert torch.allclose(infonce_loss(q, d, 0.05), ref, atol=1e-6)
    off = F.cross_entropy(q[:3] @ d.t() / 0.05, torch.arange(3) + 4)
    assert torch.allclose(infonce_loss(q[:3], d, 0.05, target_offset=4), off, atol=1e-6)


def test_topk_truncation():
    q, d = _emb(5, 8, 2), _emb(5, 8, 3)
    full = infonce_loss(q, d, 0.1)
    assert torch.allclose(infonce_loss(q, d, 0.1, top_k=4), full, atol=1e-6)  # k = all negatives
    assert infonce_loss(q, d, 0.1, top_k=2) <= full + 1e-6


def test_single_positive_label_matrix_equals_infonce():
    q, d = _emb(4, 8, 4), _emb(4, 8, 5)
    labels = torch.eye(4)
    assert torch.allclose(contrastive_loss(q, d, labels, 0.05), infonce_loss(q, d, 0.05), atol=1e-6)
    assert torch.allclose(fused_contrastive_loss(q, d, labels, 0.05), infonce_loss(q, d, 0.05), atol=1e-6)


def test_multi_positive_ignore_and_grads():
    q, d = _emb(3, 8, 6).requires_grad_(), _emb(5, 8, 7).requires_grad_()
    labels = torch.tensor([[1., 1, 0, 0, -1], [0, 0, 1, 0, 0], [0, 0, 0, 0, 0]])
    loss = contrastive_loss(q, d, labels, 0.1)
    sim = (q @ d.t()) / 0.1
    r0 = torch.logsumexp(sim[0, :4], 0) - sim[0, :2].mean()
    r1 = torch.logsumexp(sim[1], 0) - sim[1, 2]
    assert torch.allclose(loss, (r0 + r1) / 2, atol=1e-6)  # query 2 has no positive: skipped
    loss.backward()
    assert q.grad[2].abs().sum() == 0 and d.grad.abs().sum() > 0
    none = contrastive_loss(q, d, torch.zeros(3, 5), 0.1)
    assert none.item() == 0.0 and none.requires_grad


def test_soft_labels():
    q, d = _emb(2, 8, 8), _emb(3, 8, 9)
    labels = torch.tensor([[1., 0, 0], [0, 1, 0]])
    scores = torch.tensor([[3., 1, 5.0], [0., 2, 1]])
    labels[0, 2] = -1   # ignored column: its score does not count and it leaves the denominator
    loss = contrastive_loss(q, d, labels, 0.1, scores=scores)
    sim = (q @ d.t()) / 0.1
    # targets are the scores normalised to sum to one (lset/losses/contrastive.py:27-38)
    t0, lp0 = scores[0, :2] / scores[0, :2].sum(), torch.log_softmax(sim[0, :2], 0)
    t1, lp1 = scores[1] / scores[1].sum(), torch.log_softmax(sim[1], 0)
    assert torch.allclose(loss, (-(t0 * lp0).sum() - (t1 * lp1).sum()) / 2, atol=1e-6)


def test_matryoshka_and_logit_scale():
    q, d = _emb(4, 16, 10), _emb(4, 16, 11)
    l = matryoshka_loss(q, d, [4, 16], 0.05)
    parts = [infonce_loss(F.normalize(q[:, :k], dim=-1), F.normalize(d[:, :k], dim=-1), 0.05) for k in (4, 16)]
    assert torch.allclose(l, sum(parts) / 2, atol=1e-6)
    s = LogitScale.from_temperature(0.02, learnable=True)
    assert math.isclose(s().item(), 50.0, rel_tol=1e-5) and s.log_scale.requires_grad
    s.log_scale.data.fill_(10.0)
    assert s().item() == s.max_scale
    assert not LogitScale(20.0, learnable=False).log_scale.requires_grad
    assert LogitScale(20.0, 50.0).max_scale == 50.0      # positional order: init, max, learnable
    with pytest.raises(ValueError):
        LogitScale(0.0)
    with pytest.raises(ValueError):
        LogitScale.from_temperature(-1.0)


def test_task_joint_encode_equals_separate():
    from lset_b200.models import Qwen3Config, Qwen3Decoder
    from lset_b200.models.layers import init_normal_
    from lset_b200.tasks.bi_encoder import BiEncoderTask
    from lset_b200.train.data.packing import pack_sequences

    torch.manual_seed(0)
    m = Qwen3Decoder(Qwen3Config(vocab_size=100, hidden_size=32, intermediate_size=64,
                                 num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                 head_dim=8))
    init_normal_(m, 0.05)
    q = pack_sequences([[1, 2, 3], [4, 5]])
    d = pack_sequences([[6, 7, 8, 9], [10, 11, 12]])
    n = pack_sequences([[13, 14], [15, 16, 17]])
    a = BiEncoderTask(joint_encode=True)(m, q, d, n)
    b = BiEncoderTask(joint_encode=False)(m, q, d, n)
    assert torch.allclose(a["loss"], b["loss"], atol=1e-5)
    assert torch.allclose(a["query_embeds"], b["query_embeds"], atol=1e-5)
    lm = BiEncoderTask()(m, q, d, labels=torch.eye(2))
    assert torch.allclose(lm["loss"], BiEncoderTask()(m, q, d)["loss"], atol=1e-5)


def test_fused_dispatcher_follows_reference_thresholds_and_falls_back_on_cpu():
    from lset_b200.losses import fused_contrastive_loss
    from lset_b200.ops.loss import reference_switches_to_fused

    # sizes from which the reference replaces the eager label loss by its fused kernel
    assert not reference_switches_to_fused(1023, 10**6, "multi")
    assert reference_switches_to_fused(1024, 4096, "multi") and not reference_switches_to_fused(1024, 4095, "multi")
    assert reference_switches_to_fused(2048, 8, "multi")
    assert reference_switches_to_fused(2048, 4096, "soft") and not reference_switches_to_fused(4096, 4095, "cross")
    # on the CPU (no streaming kernels) the dispatcher is the label-matrix loss itself
    q, d = _emb(3, 8, 20), _emb(5, 8, 21)
    labels = torch.tensor([[1., 0, 0, -1, 0], [0, 1, 1, 0, 0], [0, 0, 0, 0, 1]])
    qi, di = (labels > 0).nonzero(as_tuple=True)
    a = fused_contrastive_loss(q, d, labels, 0.1, pos_qi=qi, pos_di=di, force_fused=True)
    b = contrastive_loss(q, d, labels, 0.1)
    assert torch.allclose(a, b)


def test_scored_batches_train_documents_of_other_samples_are_negatives():
    """The collator fills the score matrix with -inf for documents of other samples; those are
    in-batch negatives with target 0, and the loss of a scored batch is the soft-label
    cross-entropy over all documents (not identically zero)."""
    from lset_b200.losses.contrastive import contrastive_loss

    torch.manual_seed(0)
    q = torch.nn.functional.normalize(torch.randn(3, 16), dim=-1).requires_grad_()
    d = torch.nn.functional.normalize(torch.randn(6, 16), dim=-1).requires_grad_()
    labels = torch.zeros(3, 6)
    scores = torch.full((3, 6), float("-inf"))
    for i in range(3):
        labels[i, 2 * i] = 1.0
        scores[i, 2 * i], scores[i, 2 * i + 1] = 3.0, 1.0
    loss = contrastive_loss(q, d, labels, 0.05, scores=scores)
    sim = (q @ d.t()) / 0.05
    target = torch.zeros(3, 6)
    for i in range(3):
        target[i, 2 * i], target[i, 2 * i + 1] = 0.75, 0.25
    want = (torch.logsumexp(sim, dim=1) - (target * sim).sum(1)).mean()
    assert float(loss) > 0 and torch.allclose(loss, want, atol=1e-5)
    loss.backward()
    assert torch.isfinite(q.grad).all() and torch.isfinite(d.grad).all() and float(d.grad.abs().sum()) > 0
