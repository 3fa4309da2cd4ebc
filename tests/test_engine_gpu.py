"""End-to-end checks on the native kernels: training through the engine on a B200."""
import pytest
import torch

from lset_b200.models import BertConfig, GemmaConfig, LlamaConfig, Qwen3Config
from lset_b200.ops import _native as nv
from lset_b200.train.data.collator import LeftPadCollator, PackedCollator
from lset_b200.train.data.dataset import SyntheticPairDataset
from lset_b200.train.engine import TrainingEngine

pytestmark = pytest.mark.gpu


def _cfg():
    return Qwen3Config(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=128)


def _engine(device="cuda", name="qwen3", cfg=None, **kw):
    torch.manual_seed(0)
    base = dict(batch_size=8, lr=1e-3, packed=True, model_config=cfg or _cfg(), log_interval=0,
                scheduler_type="constant", fused_projections=True, device=device)
    base.update(kw)
    return TrainingEngine(name, None, None, **base)


def _batch(lo, hi, packed=True, vocab=2048):
    ds = SyntheticPairDataset(64, vocab, (8, 24), (40, 200), seed=3)
    return (PackedCollator() if packed else LeftPadCollator(0))([ds[i] for i in range(lo, hi)])


def _flat(eng):
    return torch.cat([g.flat_grad.float().cpu() for g in eng.store.groups])


@pytest.mark.parametrize("packed", [True, False])
def test_gpu_matches_cpu_oracle_and_learns(packed):
    gpu, cpu = _engine(packed=packed), _engine("cpu", packed=packed)
    lg = float(gpu.forward_backward(_batch(0, 8, packed), True))
    lc = float(cpu.forward_backward(_batch(0, 8, packed), True))
    nv.check_status()
    assert abs(lg - lc) < 0.08 * max(1.0, abs(lc)), (lg, lc)
    gg, gc = _flat(gpu), _flat(cpu)
    cos = torch.nn.functional.cosine_similarity(gg, gc, dim=0).item()
    assert cos > 0.98, cos
    # group by group (one per layer plus the root group), so that a wrong gradient in a small
    # parameter set (norm weights, q/k norms) cannot hide behind the large matrices
    for a, b in zip(gpu.store.groups, cpu.store.groups):
        ga, gb = a.flat_grad.float().cpu(), b.flat_grad.float().cpu()
        rel = ((ga - gb).norm() / gb.norm().clamp_min(1e-12)).item()
        assert rel < 3e-2, (a.name, rel)
        for p, o in zip(b.params, b.offsets):   # and every parameter on its own, more loosely
            pa, pb = ga[o:o + p.numel()], gb[o:o + p.numel()]
            prel = ((pa - pb).norm() / pb.norm().clamp_min(1e-12)).item()
            assert prel < 6e-2, (a.name, tuple(p.shape), prel)
    gpu.optimizer_step()
    losses = [float(gpu.train_step(_batch(0, 8, packed))) for _ in range(8)]
    assert losses[-1] < losses[0], losses
    assert nv.launches() > 0


def test_grad_cache_and_activation_checkpointing_on_gpu():
    ref = _engine()
    lr = float(ref.forward_backward(_batch(0, 8), True))
    for kw in (dict(use_grad_cache=True, gc_chunk_size=3, gc_token_budget=300),
               dict(activation_checkpoint=True, ac_mode="selective"),
               dict(activation_checkpoint=True, ac_mode="full")):
        eng = _engine(**kw)
        l = float(eng.forward_backward(_batch(0, 8), True))
        nv.check_status()
        assert abs(l - lr) < 2e-2 * max(1.0, abs(lr)), (kw, l, lr)
        cos = torch.nn.functional.cosine_similarity(_flat(eng), _flat(ref), dim=0).item()
        assert cos > 0.995, (kw, cos)


def test_weight_gradients_reach_main_grad_under_checkpointing(monkeypatch):
    """Checkpointing hands the backward detached aliases of the parameters; the weight gradients
    must still be accumulated straight into the fp32 buffers (nothing arrives as ``param.grad``)."""
    from lset_b200.dist.sharded import FlatGroup

    folded = []
    orig = FlatGroup.collect_autograd_grads

    def spy(self):
        folded.extend(p for p in self.params if p.grad is not None)
        return orig(self)

    monkeypatch.setattr(FlatGroup, "collect_autograd_grads", spy)
    eng = _engine(activation_checkpoint=True, ac_mode="selective")
    eng.forward_backward(_batch(0, 8), True)
    nv.check_status()
    assert not folded, f"{len(folded)} weight gradients took the autograd route"


def test_lora_on_gpu():
    eng = _engine(lora=True, lora_r=16, lora_alpha=32.0, fused_projections=False, lr=2e-3)
    base = eng.model.layers[0].mlp.down_proj.base_linear.weight.clone()
    losses = [float(eng.train_step(_batch(0, 8))) for _ in range(6)]
    nv.check_status()
    assert all(l == l for l in losses) and min(losses[1:]) < losses[0], losses
    assert torch.equal(base, eng.model.layers[0].mlp.down_proj.base_linear.weight)


@pytest.mark.parametrize("name,cfg", [
    ("llama", LlamaConfig(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                          num_attention_heads=4, num_key_value_heads=2, head_dim=64)),
    ("embeddinggemma", GemmaConfig(vocab_size=2048, hidden_size=256, intermediate_size=512,
                                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                                   head_dim=64, query_pre_attn_scalar=64,
                                   layer_types=["sliding_attention", "full_attention"])),
    ("bert", BertConfig(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                        num_attention_heads=4, max_position_embeddings=512)),
])
def test_other_families_train_on_gpu(name, cfg):
    gpu = _engine(name=name, cfg=cfg, fused_projections=False)
    cpu = _engine("cpu", name=name, cfg=cfg, fused_projections=False)
    lg = float(gpu.forward_backward(_batch(0, 8), True))
    lc = float(cpu.forward_backward(_batch(0, 8), True))
    nv.check_status()
    assert abs(lg - lc) < 0.1 * max(1.0, abs(lc)), (name, lg, lc)
    gpu.optimizer_step()
    losses = [float(gpu.train_step(_batch(0, 8))) for _ in range(6)]
    assert losses[-1] < losses[0], (name, losses)


def test_step_after_a_bounded_wait_timeout_changes_nothing_and_is_not_saved(tmp_path):
    """A kernel that gives up a bounded wait leaves a non-zero status word. The optimizer sees it on
    the device (no host sync) and applies nothing: parameters, master weights and moments stay bit
    for bit; ``save`` refuses to write such a state. The wait that runs out here is the probe
    kernel's, on a flag that nothing sets; nothing faults and the context stays usable."""
    import ctypes
    import os

    eng = _engine(output_dir=str(tmp_path))
    eng.train_step(_batch(0, 8))                       # a normal step first: moments are non-zero
    eng.forward_backward(_batch(8, 16), True)
    lib = nv.load()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    word = nv.status_word(eng.device)
    rc = lib.lb_bounded_wait_probe(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint(1),
                                   ctypes.c_ulonglong(100_000_000), ctypes.c_void_p(word.data_ptr()),
                                   ctypes.c_void_p(waited.data_ptr()),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    snap = [(g.flat_param.clone(), g.master.clone(), g.exp_avg.clone(), g.exp_avg_sq.clone())
            for g in eng.store.groups]
    eng.optimizer.step()
    torch.cuda.synchronize()
    assert int(word.item()) == 4
    for g, (p, m, a, b) in zip(eng.store.groups, snap):
        assert torch.equal(g.flat_param, p) and torch.equal(g.master, m), g.name
        assert torch.equal(g.exp_avg, a) and torch.equal(g.exp_avg_sq, b), g.name
    with pytest.raises(nv.NativeError):
        eng.save(1)
    assert not os.path.exists(tmp_path / "step_1" / "meta.pt")
    # the status word was cleared by the check: the next step trains again
    eng.optimizer.zero_grad()
    before = eng.store.groups[0].master.clone()
    eng.train_step(_batch(0, 8))
    torch.cuda.synchronize()
    assert not torch.equal(before, eng.store.groups[0].master)
    nv.check_status()
