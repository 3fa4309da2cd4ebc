"""Two data-parallel ranks (gloo) against one process on the union batch, across model families,
batch layouts and training options: the global loss and, after the reduction, every gradient must
agree. One spawn runs all variants. Parity tier of the reference's multi-model integration tests
(tests/test_multi_model_training.py), which only check that each combination runs."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lset_b200.models import BertConfig, GemmaConfig, LlamaConfig, Qwen3Config
from lset_b200.train.data.collator import LeftPadCollator, PackedCollator, RightPadCollator
from lset_b200.train.data.dataset import SyntheticPairDataset
from lset_b200.train.engine import TrainingEngine

_DEC = dict(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, head_dim=8)
_ENC = dict(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
            num_attention_heads=4, max_position_embeddings=64)
# name -> (family, config, engine options, hard negatives per pair)
VARIANTS = {
    "qwen3-padded": ("qwen3", Qwen3Config(**_DEC), dict(packed=False), 0),
    "qwen3-fused-projections": ("qwen3", Qwen3Config(**_DEC),
                                dict(packed=True, fused_projections=True), 0),
    "llama-packed": ("llama", LlamaConfig(**_DEC), dict(packed=True), 0),
    "gemma-padded": ("embeddinggemma",
                     GemmaConfig(sliding_window=64, query_pre_attn_scalar=8, **_DEC),
                     dict(packed=False), 0),
    "bert-padded-negatives": ("bert", BertConfig(**_ENC), dict(packed=False), 1),
    "qlora-packed": ("qwen3", Qwen3Config(**_DEC),
                     dict(packed=True, qlora=True, lora_r=4, qlora_block_size=16), 0),
    "lora-padded-gradcache": ("qwen3", Qwen3Config(**_DEC),
                              dict(packed=False, lora=True, lora_r=4, use_grad_cache=True,
                                   gc_chunk_size=2), 1),
    "accumulation": ("qwen3", Qwen3Config(**_DEC),
                     dict(packed=True, gradient_accumulation_steps=2), 0),
    "learnable-temperature": ("qwen3", Qwen3Config(**_DEC),
                              dict(packed=True, learnable_temperature=True), 3),
    "matryoshka": ("qwen3", Qwen3Config(**_DEC),
                        dict(packed=True, matryoshka_dims=[8, 16, 32]), 0),
    "full-recompute": ("qwen3", Qwen3Config(**_DEC),
                       dict(packed=True, activation_checkpoint=True, ac_mode="full"), 0),
    # parameter-sharded mode (layers hold 1/W of parameters and gradients) with other options
    "sharded-padded-recompute": ("qwen3", Qwen3Config(**_DEC),
                                 dict(packed=False, reshard_after_forward=True,
                                      activation_checkpoint=True, ac_mode="full"), 1),
    "sharded-gradcache-accumulation": ("qwen3", Qwen3Config(**_DEC),
                                       dict(packed=True, reshard_after_forward=True,
                                            use_grad_cache=True, gc_chunk_size=2,
                                            gradient_accumulation_steps=2), 0),
}


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _engine(family, cfg, opts, dp):
    torch.manual_seed(0)
    return TrainingEngine(family, None, None, dp_size=dp, batch_size=8 // dp, lr=1e-2,
                          model_config=cfg, log_interval=0, device="cpu", grad_clip=0.0,
                          scheduler_type="constant", **opts)


def _batch(lo, hi, family, packed, negs):
    ds = SyntheticPairDataset(16, 300, (3, 6), (5, 12), seed=5, num_negatives=negs)
    if packed:
        coll = PackedCollator()
    else:
        coll = RightPadCollator(0) if family == "bert" else LeftPadCollator(0)
    return coll([ds[i] for i in range(lo, hi)])


def _gradients(family, cfg, opts, negs, dp, rank):
    eng = _engine(family, cfg, opts, dp)
    per = 8 // dp
    micro = opts.get("gradient_accumulation_steps", 1)
    for m in range(micro):
        lo = 8 * m + rank * per
        loss = eng.forward_backward(_batch(lo, lo + per, family, opts["packed"], negs), m == micro - 1)
    return eng, loss


def _worker(rank, world, port, out_path):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    res = {}
    for name, (family, cfg, opts, negs) in VARIANTS.items():
        eng, loss = _gradients(family, cfg, opts, negs, world, rank)
        total = loss.clone()
        dist.all_reduce(total)
        stores = [eng.store] + ([eng.task_store] if eng.task_store is not None else [])
        if opts.get("reshard_after_forward"):
            assert eng.store.zero3
        res[name] = (float(total), [[st._gather_fp32(g, g.grad_shard) for g in st.groups]
                                    for st in stores])
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.fixture(scope="module")
def two_rank_results():
    out_path = os.path.join(tempfile.mkdtemp(), "dp2.pt")
    mp.spawn(_worker, args=(2, _port(), out_path), nprocs=2, join=True)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        os.environ.pop(k, None)
    return torch.load(out_path, weights_only=False)


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_two_ranks_agree_with_one_process(two_rank_results, name):
    family, cfg, opts, negs = VARIANTS[name]
    total, grads = two_rank_results[name]
    eng, loss = _gradients(family, cfg, opts, negs, 1, 0)
    assert float(loss) == pytest.approx(total, abs=2e-4)
    stores = [eng.store] + ([eng.task_store] if eng.task_store is not None else [])
    assert len(stores) == len(grads)
    for st, per_store in zip(stores, grads):
        assert len(st.groups) == len(per_store)
        for g, ref in zip(st.groups, per_store):
            n = min(g.flat_grad.numel(), ref.numel())   # the gathered copy is padded to the shards
            # the data-parallel average of the ranks' gradients = union-batch gradient / world
            diff = (g.flat_grad[:n] / 2 - ref[:n]).abs().max()
            assert float(diff) < 5e-5 * max(1.0, float(ref.abs().max())), (name, float(diff))
