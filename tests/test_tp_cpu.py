"""Tensor parallelism on CPU (gloo, 2 ranks): sharded forward and gradients equal the unsharded
model's; plan structure; gradient norm across tensor-parallel shards."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lset_b200.models import Qwen3Config, Qwen3Decoder
from lset_b200.models.layers import init_normal_
from lset_b200.models.parallel_plan import bert_tp_plan, decoder_tp_plan


def _cfg():
    return Qwen3Config(vocab_size=200, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=8)


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir, fused, sp=False):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lset_b200.dist.tp import apply_tp

    torch.manual_seed(0)
    m = Qwen3Decoder(_cfg(), fused_projections=fused)
    init_normal_(m, 0.05)
    full = {k: v.clone() for k, v in m.state_dict().items()}
    apply_tp(m, dist.group.WORLD, decoder_tp_plan(_cfg(), fused_projections=fused,
                                                  use_sequence_parallel=sp))
    # data-parallel world of one per rank: the store only has to sum the partial gradients of the
    # per-head norm weights over the tensor-parallel group
    from lset_b200.dist.sharded import ParamStore

    dp_groups = [dist.new_group([r]) for r in range(world)]
    store = ParamStore(m, dp_group=dp_groups[rank], compute_dtype=torch.float32,
                       device=torch.device("cpu"), tp_group=dist.group.WORLD)
    ids = _ids(sp)
    out = m(ids)["hidden_states"]
    out.pow(2).sum().backward()
    store.finish_backward()
    params = dict(m.named_parameters())
    g = params["layers.0.mlp.down_proj.weight"].main_grad.clone()
    gq = params["layers.0.self_attn.q_norm.weight"].main_grad.clone()
    gk = params["layers.1.self_attn.k_norm.weight"].main_grad.clone()
    gn = params["layers.1.input_layernorm.weight"].main_grad.clone()
    ge = params["embed_tokens.weight"].main_grad.clone()
    if rank == 0:
        torch.save({"out": out.detach(), "grad": g, "gq": gq, "gk": gk, "gn": gn, "ge": ge,
                    "full": full},
                   os.path.join(out_dir, "tp.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _ids(sp):
    # 15 tokens under sequence parallelism: not a multiple of the group size, so padding is covered
    return (torch.arange(15).reshape(3, 5) if sp else torch.arange(14).reshape(2, 7)) % 200


@pytest.mark.parametrize("fused,sp", [(False, False), (True, False), (False, True), (True, True)])
def test_tp_matches_unsharded(fused, sp):
    out_dir = tempfile.mkdtemp()
    mp.spawn(_worker, args=(2, _port(), out_dir, fused, sp), nprocs=2, join=True)
    got = torch.load(os.path.join(out_dir, "tp.pt"), weights_only=False)
    ref = Qwen3Decoder(_cfg(), fused_projections=fused)
    ref.load_state_dict(got["full"])
    ids = _ids(sp)
    out = ref(ids)["hidden_states"]
    out.pow(2).sum().backward()
    assert torch.allclose(out, got["out"], atol=1e-5), (out - got["out"]).abs().max()
    gfull = ref.layers[0].mlp.down_proj.weight.grad
    assert torch.allclose(gfull[:, :32], got["grad"], atol=1e-4)  # rank 0 owns the first half of the inputs
    # per-head norm weights: each rank sees only its heads, the store sums the partial gradients
    assert torch.allclose(ref.layers[0].self_attn.q_norm.weight.grad, got["gq"], atol=1e-4)
    assert torch.allclose(ref.layers[1].self_attn.k_norm.weight.grad, got["gk"], atol=1e-4)
    # token-sharded norms (sequence parallelism) and the embedding see the full gradient too
    assert torch.allclose(ref.layers[1].input_layernorm.weight.grad, got["gn"], atol=1e-4)
    assert torch.allclose(ref.embed_tokens.weight.grad, got["ge"], atol=1e-4)


def _fp8_worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lset_b200.dist.tp import apply_tp
    from lset_b200.train.quantization.fp8 import Float8Linear, apply_fp8_training

    torch.manual_seed(0)
    m = Qwen3Decoder(_cfg(), fused_projections=False)
    init_normal_(m, 0.05)
    full = {k: v.clone() for k, v in m.state_dict().items()}
    apply_fp8_training(m, "tensorwise")      # the engine's order: fp8 first, then the TP plan
    apply_tp(m, dist.group.WORLD, decoder_tp_plan(_cfg()))
    n_fp8 = sum(isinstance(x, Float8Linear) for x in m.modules())
    out = m(_ids(False))["hidden_states"]
    out.pow(2).sum().backward()
    g = m.layers[0].mlp.down_proj.weight.grad.clone()
    if rank == 0:
        torch.save({"out": out.detach(), "grad": g, "full": full, "n_fp8": n_fp8},
                   os.path.join(out_dir, "tp_fp8.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_tp_with_fp8_linears():
    """FP8 linear layers keep working under the all-reduce tensor-parallel scheme: shards are
    quantised per rank, so the result is fp8-close (not equal) to the unsharded full-precision model."""
    out_dir = tempfile.mkdtemp()
    mp.spawn(_fp8_worker, args=(2, _port(), out_dir), nprocs=2, join=True)
    got = torch.load(os.path.join(out_dir, "tp_fp8.pt"), weights_only=False)
    assert got["n_fp8"] >= 12
    ref = Qwen3Decoder(_cfg(), fused_projections=False)
    ref.load_state_dict(got["full"])
    out = ref(_ids(False))["hidden_states"]
    out.pow(2).sum().backward()
    rel = lambda a, b: float((a - b).abs().max() / b.abs().max())  # noqa: E731
    assert rel(got["out"], out.detach()) < 0.15
    assert rel(got["grad"], ref.layers[0].mlp.down_proj.weight.grad[:, :32]) < 0.3


def test_plans():
    p = decoder_tp_plan(None)
    assert p["layers.*.self_attn.q_proj"] == "colwise" and p["layers.*.mlp.down_proj"] == "rowwise"
    pf = decoder_tp_plan(None, fused_projections=True)
    assert "layers.*.self_attn.qkv_proj" in pf and "layers.*.mlp.gate_up_proj" in pf
    pl = decoder_tp_plan(None, use_lora=True)
    assert pl["layers.*.self_attn.q_proj.lora_B"] == "colwise"
    assert pl["layers.*.self_attn.o_proj.lora_A"] == "rowwise"
    ps = decoder_tp_plan(None, use_sequence_parallel=True)
    assert ps["norm"] == "sequence"
    assert decoder_tp_plan(None, use_sequence_parallel=True, use_lora=True).get("norm") is None
    pb = bert_tp_plan(None)
    assert pb["layers.*.attention.query"] == "colwise" and pb["layers.*.mlp.dense_out"] == "rowwise"


def _lora_traj(tp):
    from lset_b200.tasks.bi_encoder import global_loss_value
    from lset_b200.train.data.collator import PackedCollator
    from lset_b200.train.data.dataset import SyntheticPairDataset
    from lset_b200.train.engine import TrainingEngine

    torch.manual_seed(0)
    cfg = Qwen3Config(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=8)
    eng = TrainingEngine("qwen3", None, None, dp_size=1, tp_size=tp, batch_size=8, lr=3e-3,
                         packed=True, model_config=cfg, log_interval=0, device="cpu", grad_clip=1.0,
                         scheduler_type="constant", lora=True, lora_r=4)
    ds = SyntheticPairDataset(16, 300, (3, 6), (5, 12), seed=5)
    coll = PackedCollator()
    out = []
    for s in range(3):
        lo = (s % 2) * 8
        loss = eng.train_step(coll([ds[i] for i in range(lo, lo + 8)]))
        out.append(float(global_loss_value(loss, eng.dp_group)))
    return out


def _lora_worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    losses = _lora_traj(world)
    if rank == 0:
        torch.save(losses, os.path.join(out_dir, "lora_tp.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_lora_under_tensor_parallelism_trains_like_one_process():
    """Adapters on column-parallel layers: ``lora_B`` is column-sharded and its rank-r input is
    replicated, so the gradient flowing back into that input (and with it ``lora_A``'s weight
    gradient and the adapter's share of dx) is a partial sum per rank until it is all-reduced.
    The third loss depends on ``lora_A``'s second gradient (its first one is zero because
    ``lora_B`` starts at zero)."""
    out_dir = tempfile.mkdtemp()
    mp.spawn(_lora_worker, args=(2, _port(), out_dir), nprocs=2, join=True)
    got = torch.load(os.path.join(out_dir, "lora_tp.pt"), weights_only=False)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        os.environ.pop(k, None)
    ref = _lora_traj(1)
    assert got == pytest.approx(ref, abs=1e-4), (got, ref)
