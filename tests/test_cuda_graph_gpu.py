"""CUDA-graph capture of the model forward: replay must reproduce the eager forward on batches
other than the one that was captured (cf. the reference's tests/train/test_cuda_graph.py)."""
import pytest
import torch

from lset_b200.models import Qwen3Config
from lset_b200.models.decoder import Qwen3Decoder
from lset_b200.ops import _native as nv
from lset_b200.train.cuda_graph import CUDAGraphWrapper, PackedCUDAGraphWrapper
from lset_b200.train.data.collator import FixedBudgetPackedCollator

pytestmark = pytest.mark.gpu


def _model():
    torch.manual_seed(0)
    cfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    m = Qwen3Decoder(cfg, fused_projections=True)
    for p in m.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.05)
    return m.cuda().to(torch.bfloat16).eval()


def test_padded_graph_replay_matches_eager_on_new_batches():
    model = _model()
    wrap = CUDAGraphWrapper(model, batch_size=4, seq_length=48, device="cuda")
    g = torch.Generator().manual_seed(1)
    for _ in range(2):
        ids = torch.randint(0, 512, (4, 48), generator=g).cuda()
        got = wrap(ids)["hidden_states"].clone()
        with torch.no_grad():
            want = model(ids)["hidden_states"]
        assert torch.equal(got, want)
    nv.check_status()


def test_packed_fixed_budget_graph_replay_matches_eager_on_new_batches():
    model = _model()
    budget, max_seqs = 512, 12
    wrap = PackedCUDAGraphWrapper(model, budget, max_seqs, "cuda", max_seqlen=128)
    coll = FixedBudgetPackedCollator(token_budget=budget)
    g = torch.Generator().manual_seed(2)
    for n_seq in (5, 9):
        lens = torch.randint(8, 56, (n_seq,), generator=g).tolist()
        samples = [{"query": {"input_ids": torch.randint(1, 512, (n,), generator=g).tolist()},
                    "positive": {"input_ids": [1, 2, 3]}} for n in lens]
        batch = coll(samples)["query"]
        batch = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in batch.items()}
        total = int(batch["cu_seqlens"][-1])
        got = wrap(batch)["hidden_states"][:total].clone()
        with torch.no_grad():
            want = model(batch["input_ids"], position_ids=batch["position_ids"],
                         cu_seqlens=batch["cu_seqlens"], max_seqlen=128)["hidden_states"][:total]
        assert torch.equal(got, want)
    nv.check_status()
