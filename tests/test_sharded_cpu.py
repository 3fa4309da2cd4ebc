"""Sharded data parallelism on CPU (gloo, 2 ranks): gradients, loss and updated weights agree with
a single process that sees the union batch; checkpoint state round-trips."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lset_b200.models import Qwen3Config
from lset_b200.train.data.collator import PackedCollator
from lset_b200.train.data.dataset import SyntheticPairDataset
from lset_b200.train.engine import TrainingEngine


def _cfg():
    return Qwen3Config(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _engine(dp, **kw):
    torch.manual_seed(0)
    return TrainingEngine("qwen3", None, None, dp_size=dp, batch_size=4, lr=1e-2, packed=True,
                          model_config=_cfg(), log_interval=0, device="cpu", grad_clip=0.0,
                          scheduler_type="constant", **kw)


def _batch(lo, hi):
    ds = SyntheticPairDataset(16, 300, (3, 6), (5, 12), seed=5)
    return PackedCollator()([ds[i] for i in range(lo, hi)])


def _worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    eng = _engine(world, output_dir=os.path.join(out_dir, "ckpt"))
    loss = eng.forward_backward(_batch(rank * 4, rank * 4 + 4), True)
    total = loss.clone()
    dist.all_reduce(total)
    grads = [eng.store._gather_fp32(g, g.grad_shard) for g in eng.store.groups]
    eng.optimizer_step()
    params = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    eng.save(1)   # the distributed checkpoint path (sharded optimizer state)
    # round trip under sharding: train on, load the checkpoint back, state equals the saved state
    from lset_b200.train.checkpoint import latest_checkpoint, load_checkpoint

    m_saved = [g.exp_avg.clone() for g in eng.store.groups]
    eng.train_step(_batch(8 + rank * 4, 12 + rank * 4))
    moved = max(float((p.detach() - params[n]).abs().max()) for n, p in eng.model.named_parameters())
    ckpt = latest_checkpoint(os.path.join(out_dir, "ckpt"))
    step = load_checkpoint(eng.model, eng.optimizer, ckpt, store=eng.store)
    back = max(float((p.detach() - params[n]).abs().max()) for n, p in eng.model.named_parameters())
    m_back = max(float((g.exp_avg - m).abs().max()) for g, m in zip(eng.store.groups, m_saved))
    roundtrip = {"step": step, "moved": moved, "back": back, "m_back": m_back,
                 "steps_seen": eng.optimizer.step_count}
    if rank == 0:
        torch.save({"loss": total, "grads": grads, "params": params, "roundtrip": roundtrip},
                   os.path.join(out_dir, "dp.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_match_single_process():
    out_dir = tempfile.mkdtemp()
    port = _free_port()
    os.environ["LSET_TEST_OUT"] = out_dir
    mp.spawn(_worker, args=(2, port, out_dir), nprocs=2, join=True)
    got = torch.load(os.path.join(out_dir, "dp.pt"), weights_only=False)

    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        os.environ.pop(k, None)
    eng = _engine(1)
    # single process on the union batch: queries 0..7 against documents 0..7
    loss = eng.forward_backward(_batch(0, 8), True)
    assert torch.allclose(loss, got["loss"], atol=1e-5), (loss, got["loss"])
    for g, ref in zip(eng.store.groups, got["grads"]):
        # data-parallel mean of per-rank gradients = union-batch gradient / world
        assert torch.allclose(g.flat_grad / 2, ref, atol=2e-5), (g.flat_grad / 2 - ref).abs().max()
    rt = got["roundtrip"]
    assert rt["step"] == 1 and rt["moved"] > 1e-4 and rt["back"] < 1e-6 and rt["m_back"] < 1e-7, rt
    assert rt["steps_seen"] == 1        # the optimizer's step counter came back with the state


def _zero3_worker(rank, world, port, out_dir, zero3):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    eng = _engine(world, reshard_after_forward=zero3, gradient_accumulation_steps=2)
    losses = []
    for s in range(4):                      # two optimizer steps of two micro-steps each
        lo = (s % 2) * 8 + rank * 4
        loss = eng.train_step(_batch(lo, lo + 4)).clone()
        dist.all_reduce(loss)
        losses.append(float(loss))
    masters = {n: t.clone() for n, t in eng.store.named_master_tensors()}
    # evaluation forward after training: the layers gather their parameters on demand
    with torch.no_grad():
        b = _batch(0, 4)["query"]
        hid = eng.model.forward_packed(b["input_ids"], b["position_ids"], b["cu_seqlens"],
                                       b["max_seqlen"])["hidden_states"].clone()
    if rank == 0:
        torch.save({"losses": losses, "masters": masters, "hidden": hid,
                    "memory": eng.store.memory_report(), "zero3": eng.store.zero3},
                   os.path.join(out_dir, f"z{int(zero3)}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_parameter_sharded_mode_matches_resident_mode():
    """``reshard_after_forward`` (layers keep 1/W of parameters and gradients; full copies live in
    rotating buffers gathered per layer) trains exactly like the resident-replica mode, gradient
    accumulation included, and holds about half the layer state per rank at two ranks."""
    out_dir = tempfile.mkdtemp()
    for zero3 in (False, True):
        mp.spawn(_zero3_worker, args=(2, _free_port(), out_dir, zero3), nprocs=2, join=True)
    a = torch.load(os.path.join(out_dir, "z0.pt"), weights_only=False)
    b = torch.load(os.path.join(out_dir, "z1.pt"), weights_only=False)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        os.environ.pop(k, None)
    assert not a["zero3"] and b["zero3"]
    assert a["losses"] == pytest.approx(b["losses"], abs=1e-5)
    for n, t in a["masters"].items():
        assert torch.allclose(t, b["masters"][n], atol=1e-6), n
    assert torch.allclose(a["hidden"], b["hidden"], atol=1e-5)
    ma, mb = a["memory"], b["memory"]
    assert mb["sharded_groups"] == 2 and ma["sharded_groups"] == 0
    # the root group (embeddings) stays resident in both; everything else halves
    assert mb["param_bytes"] < ma["param_bytes"] and mb["grad_bytes"] < ma["grad_bytes"]
    assert mb["optim_bytes"] == ma["optim_bytes"]


def _padded_worker(rank, world, port, out_dir):
    from lset_b200.train.data.collator import LeftPadCollator

    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ds = SyntheticPairDataset(16, 300, (3, 6), (5, 12), seed=5)
    res = {}
    for packed in (True, False):
        torch.manual_seed(0)
        eng = TrainingEngine("qwen3", None, None, dp_size=world, batch_size=4, lr=1e-2,
                             packed=packed, model_config=_cfg(), log_interval=0, device="cpu",
                             grad_clip=1.0, scheduler_type="constant")
        collate = PackedCollator() if packed else LeftPadCollator(0)
        losses = []
        for s in range(3):
            lo = (s % 2) * 8 + rank * 4
            losses.append(float(eng.train_step(collate([ds[i] for i in range(lo, lo + 4)]))))
        res[packed] = {"losses": losses,
                       "masters": {n: t.clone() for n, t in eng.store.named_master_tensors()}}
    if rank == 0:
        torch.save(res, os.path.join(out_dir, "padded.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_layers_run_twice_per_step_reduce_after_the_last_pass():
    """Padded batches encode queries and documents in separate passes, so every layer's backward
    hook fires twice inside one ``backward()``: the gradient reduction of a layer must wait for
    the second. Two ranks on padded batches train exactly like two ranks on the packed form of
    the same batches (one joint pass)."""
    out_dir = tempfile.mkdtemp()
    mp.spawn(_padded_worker, args=(2, _free_port(), out_dir), nprocs=2, join=True)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        os.environ.pop(k, None)
    res = torch.load(os.path.join(out_dir, "padded.pt"), weights_only=False)
    assert res[True]["losses"] == pytest.approx(res[False]["losses"], abs=1e-3)
    for n, t in res[True]["masters"].items():
        # Adam turns rounding noise in a near-zero gradient entry into a visible step (a rarely
        # seen embedding row), so a handful of elements may differ; a missed reduction moves all
        off = ((t - res[False]["masters"][n]).abs() > 1e-4).float().mean()
        assert off < 1e-3, (n, float(off))


def _lora_worker(rank, world, port, out_dir, grad_cache):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    eng = _engine(world, lora=True, lora_r=4, use_grad_cache=grad_cache, gc_chunk_size=2)
    loss = eng.forward_backward(_batch(rank * 4, rank * 4 + 4), True)
    total = loss.clone()
    dist.all_reduce(total)
    grads = [eng.store._gather_fp32(g, g.grad_shard) for g in eng.store.groups]
    if rank == 0:
        torch.save({"loss": total, "grads": grads},
                   os.path.join(out_dir, f"lora_{int(grad_cache)}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("grad_cache", [False, True])
def test_first_block_behind_frozen_embeddings_is_reduced_after_its_backward(grad_cache):
    """With adapters the embeddings are frozen, so no input of the first block requires a gradient
    and torch fires that block's backward hook *before* its parameters have their gradients. The
    block's gradients must still be averaged over the ranks: two ranks agree with a single process
    on the union batch, with and without GradCache."""
    out_dir = tempfile.mkdtemp()
    mp.spawn(_lora_worker, args=(2, _free_port(), out_dir, grad_cache), nprocs=2, join=True)
    got = torch.load(os.path.join(out_dir, f"lora_{int(grad_cache)}.pt"), weights_only=False)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        os.environ.pop(k, None)
    eng = _engine(1, lora=True, lora_r=4)
    loss = eng.forward_backward(_batch(0, 8), True)
    assert torch.allclose(loss, got["loss"], atol=1e-5), (loss, got["loss"])
    assert len(eng.store.groups) == len(got["grads"]) and len(got["grads"]) >= 2
    for g, ref in zip(eng.store.groups, got["grads"]):
        assert float(g.flat_grad.abs().max()) > 0
        assert torch.allclose(g.flat_grad / 2, ref, atol=2e-5), (g.flat_grad / 2 - ref).abs().max()
