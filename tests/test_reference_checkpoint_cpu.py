"""Checkpoint interchange with the reference implementation (single-process ``checkpoint.pt``):
a directory written by the reference's ``save_checkpoint`` loads into this framework's engine, and
one written here loads through the reference's ``load_checkpoint``. Needs the reference package
under ``baseline/_ref`` (installed offline from its source tree); skipped when it is absent."""
import os
import sys

import pytest
import torch

REF_ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF_ROOT, "lset")),
                                reason="reference package not installed under baseline/_ref")

DIMS = dict(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, head_dim=16)


def _reference():
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    from lset.models import get_model_spec
    from lset.train import checkpoint as ref_ckpt

    spec = get_model_spec("qwen3")
    torch.manual_seed(7)
    model = spec.model_cls(spec.config_cls(**DIMS))
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=1e-3, weight_decay=0.01)
    return model, opt, ref_ckpt


def _engine(tmp_path, fused=False):
    from lset_b200.models import Qwen3Config
    from lset_b200.train.engine import TrainingEngine

    return TrainingEngine("qwen3", None, None, batch_size=4, lr=1e-3, packed=True,
                          model_config=Qwen3Config(**DIMS), log_interval=0, device="cpu",
                          scheduler_type="constant", output_dir=str(tmp_path / "ours"),
                          fused_projections=fused)


def _saved_view(eng):
    """Weights and optimizer state as this engine writes them (the reference's names and
    numbering, whether its projections are fused or not)."""
    from lset_b200.train.checkpoint import model_state, optimizer_state

    return model_state(eng.model, eng.store), optimizer_state(eng.optimizer, eng.model, eng.store)["state"]


def _step_with_random_grads(model, opt, seed):
    g = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        p.grad = torch.randn(p.shape, generator=g) * 0.1
    opt.step()
    opt.zero_grad()


@pytest.mark.parametrize("fused", [False, True], ids=["unfused", "fused-projections"])
def test_reference_checkpoint_loads_into_this_engine(tmp_path, fused):
    from lset_b200.train.checkpoint import load_checkpoint

    ref_model, ref_opt, ref_ckpt = _reference()
    _step_with_random_grads(ref_model, ref_opt, 1)
    ref_ckpt.save_checkpoint(ref_model, ref_opt, 3, str(tmp_path / "ref"))
    eng = _engine(tmp_path, fused)
    step = load_checkpoint(eng.model, eng.optimizer, str(tmp_path / "ref" / "step_3"), store=eng.store)
    assert step == 3
    ours, sd = _saved_view(eng)
    for name, p in ref_model.named_parameters():
        assert torch.equal(ours[name], p.detach()), name
    ref_sd = ref_opt.state_dict()["state"]
    assert len(sd) == len(ref_sd)
    for idx, ent in ref_sd.items():
        assert torch.equal(sd[idx]["exp_avg"], ent["exp_avg"]), idx
        assert torch.equal(sd[idx]["exp_avg_sq"], ent["exp_avg_sq"]), idx
    assert eng.optimizer.step_count == 1


@pytest.mark.parametrize("fused", [False, True], ids=["unfused", "fused-projections"])
def test_checkpoint_written_here_loads_through_the_reference(tmp_path, fused):
    from lset_b200.train.data.collator import PackedCollator
    from lset_b200.train.data.dataset import SyntheticPairDataset

    eng = _engine(tmp_path, fused)
    ds = SyntheticPairDataset(8, 64, (4, 8), (8, 16), seed=0)
    eng.train_step(PackedCollator()([ds[i] for i in range(4)]))
    path = eng.save(1)
    ref_model, ref_opt, ref_ckpt = _reference()
    _step_with_random_grads(ref_model, ref_opt, 2)     # gives the optimizer a state to overwrite
    step = ref_ckpt.load_checkpoint(ref_model, ref_opt, path)
    assert step == 1
    ours, ours_opt = _saved_view(eng)
    for name, p in ref_model.named_parameters():
        assert torch.equal(p.detach(), ours[name]), name
    for idx, ent in ref_opt.state_dict()["state"].items():
        assert torch.equal(ent["exp_avg"], ours_opt[idx]["exp_avg"]), idx
        assert float(ent["step"]) == 1.0
    # and the reference optimizer can take a step from the loaded state
    _step_with_random_grads(ref_model, ref_opt, 3)
