"""Pipeline-parallel runner on CPU (gloo, 2 and 3 stages): embeddings, loss and every parameter
gradient equal the unsplit model's; split helpers agree with the runner's layer ranges."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lset_b200.dist.pp import get_pp_split_points, get_stage_module_names, stage_layer_range
from lset_b200.models import LlamaBidirectionalModel, LlamaConfig, Qwen3Config, Qwen3Decoder
from lset_b200.models.layers import init_normal_


def _cfg():
    return Qwen3Config(vocab_size=200, hidden_size=32, intermediate_size=64, num_hidden_layers=5,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=8)


def _build(family):
    if family == "llama":      # bidirectional attention, no per-head norms
        return LlamaBidirectionalModel(LlamaConfig(
            vocab_size=200, hidden_size=32, intermediate_size=64, num_hidden_layers=5,
            num_attention_heads=4, num_key_value_heads=2, head_dim=8))
    return Qwen3Decoder(_cfg())


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _microbatches():
    """Two packed micro-batches (queries, documents) and one padded one."""
    def packed(lens, off):
        ids = (torch.arange(sum(lens)) * 7 + off) % 200
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
        pos = torch.cat([torch.arange(n) for n in lens])
        return {"input_ids": ids, "cu_seqlens": cu, "position_ids": pos, "max_seqlen": max(lens)}

    return [packed([5, 3, 6], 1), packed([9, 4, 7], 11),
            {"input_ids": (torch.arange(12).reshape(3, 4) * 3) % 200}]


def _loss(hiddens, mbs):
    """InfoNCE between the last-token embeddings of micro-batch 0 and 1, plus a term on the
    padded micro-batch, so that every micro-batch's gradient depends on the others."""
    last = lambda h, mb: h[mb["cu_seqlens"][1:].long() - 1]  # noqa: E731
    q = torch.nn.functional.normalize(last(hiddens[0], mbs[0]), dim=-1)
    d = torch.nn.functional.normalize(last(hiddens[1], mbs[1]), dim=-1)
    ce = torch.nn.functional.cross_entropy(q @ d.t() / 0.05, torch.arange(q.shape[0]))
    return ce + hiddens[2].pow(2).mean()


def _worker(rank, world, port, out_dir, family="qwen3"):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lset_b200.dist.pp import PipelineRunner

    torch.manual_seed(0)
    m = _build(family)
    init_normal_(m, 0.05)
    full = {k: v.clone() for k, v in m.state_dict().items()}
    runner = PipelineRunner(m, dist.group.WORLD)
    mbs = _microbatches()
    hiddens = runner.encode(mbs)
    loss = None
    if runner.last:
        leaves = [h.detach().requires_grad_() for h in hiddens]
        loss = _loss(leaves, mbs)
        loss.backward()
        runner.backward([t.grad for t in leaves])
    else:
        assert hiddens == []
        runner.backward()
    grads = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    torch.save({"grads": grads, "full": full, "loss": None if loss is None else loss.detach(),
                "range": (runner.lo, runner.hi)}, os.path.join(out_dir, f"pp{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("stages,family", [(2, "qwen3"), (3, "qwen3"), (2, "llama")])
def test_pipeline_matches_unsplit_model(stages, family):
    out_dir = tempfile.mkdtemp()
    mp.spawn(_worker, args=(stages, _port(), out_dir, family), nprocs=stages, join=True)
    got = [torch.load(os.path.join(out_dir, f"pp{r}.pt"), weights_only=False) for r in range(stages)]
    ref = _build(family)
    ref.load_state_dict(got[0]["full"])
    mbs = _microbatches()
    hiddens = [ref(**mb)["hidden_states"] for mb in mbs]
    loss = _loss(hiddens, mbs)
    loss.backward()
    assert torch.allclose(got[-1]["loss"], loss.detach(), atol=1e-5)
    ref_grads = {n: p.grad for n, p in ref.named_parameters()}
    seen = set()
    for r, g in enumerate(got):
        lo, hi = g["range"]
        assert (lo, hi) == stage_layer_range(5, stages, r)
        for name, grad in g["grads"].items():
            assert torch.allclose(grad, ref_grads[name], atol=1e-5), name
            seen.add(name)
        owned = {n for n in g["grads"] if n.startswith("layers.")}
        assert {int(n.split(".")[1]) for n in owned} == set(range(lo, hi))
    assert seen == set(ref_grads)          # every parameter lives on exactly one stage


def test_split_helpers_agree_with_ranges():
    for n, pp in [(5, 2), (5, 3), (28, 4), (36, 8)]:
        names = get_stage_module_names(n, pp)
        points = get_pp_split_points(n, pp)
        for s in range(pp):
            lo, hi = stage_layer_range(n, pp, s)
            layers = [x for x in names[s] if x.startswith("layers.")]
            assert layers == [f"layers.{i}" for i in range(lo, hi)]
            if s > 0:
                assert points[f"layers.{lo}"] == "BEGINNING"
        assert len(points) == pp - 1


def _mesh_worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lset_b200.dist.mesh import build_mesh

    m2 = build_mesh(dp_size=2, tp_size=2, device_type="cpu")
    m3 = build_mesh(dp_size=1, tp_size=2, pp_size=2, device_type="cpu")
    info = {"names2": m2.mesh_dim_names, "names3": m3.mesh_dim_names,
            "tp2": dist.get_process_group_ranks(m2.get_group("tp")),
            "dp2": dist.get_process_group_ranks(m2.get_group("dp")),
            "pp3": dist.get_process_group_ranks(m3.get_group("pp")),
            "tp3": dist.get_process_group_ranks(m3.get_group("tp"))}
    # a collective over the tensor-parallel sub-group only sums its two members
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=m2.get_group("tp"))
    info["tp_sum"] = float(t)
    torch.save(info, os.path.join(out_dir, f"mesh{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_mesh_layout_tp_innermost_pp_outermost():
    out_dir = tempfile.mkdtemp()
    mp.spawn(_mesh_worker, args=(4, _port(), out_dir), nprocs=4, join=True)
    got = [torch.load(os.path.join(out_dir, f"mesh{r}.pt"), weights_only=False) for r in range(4)]
    assert got[0]["names2"] == ("dp", "tp") and got[0]["names3"] == ("pp", "dp", "tp")
    assert [g["tp2"] for g in got] == [[0, 1], [0, 1], [2, 3], [2, 3]]     # neighbours share TP
    assert [g["dp2"] for g in got] == [[0, 2], [1, 3], [0, 2], [1, 3]]
    assert [g["pp3"] for g in got] == [[0, 2], [1, 3], [0, 2], [1, 3]]
    assert [g["tp3"] for g in got] == [[0, 1], [0, 1], [2, 3], [2, 3]]
    assert [g["tp_sum"] for g in got] == [1.0, 1.0, 5.0, 5.0]


def _train_worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lset_b200.dist.pp import PipelineRunner
    from lset_b200.dist.sharded import ParamStore, ShardedAdamW

    torch.manual_seed(0)
    m = _build("qwen3")
    init_normal_(m, 0.05)
    runner = PipelineRunner(m, dist.group.WORLD)
    # new_group is collective: every rank creates every group, in the same order
    solo = [dist.new_group([r]) for r in range(world)][rank]
    store = ParamStore(m, dp_group=solo, compute_dtype=torch.float32, device=torch.device("cpu"))
    opt = ShardedAdamW(store, lr=1e-2, weight_decay=0.0)
    mbs, losses = _microbatches(), []
    for _ in range(3):
        hiddens = runner.encode(mbs)
        if runner.last:
            leaves = [h.detach().requires_grad_() for h in hiddens]
            loss = _loss(leaves, mbs)
            loss.backward()
            runner.backward([t.grad for t in leaves])
            losses.append(float(loss.detach()))
        else:
            runner.backward()
        store.finish_backward()
        opt.step()
        opt.zero_grad()
    if runner.last:
        torch.save(losses, os.path.join(out_dir, "pp_losses.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_pipeline_stages_train_like_the_unsplit_model():
    """Each stage owns the optimizer state of its layers: three AdamW steps through the pipeline
    give the loss trajectory of the same optimizer on the unsplit model."""
    from lset_b200.dist.sharded import ParamStore, ShardedAdamW

    out_dir = tempfile.mkdtemp()
    mp.spawn(_train_worker, args=(2, _port(), out_dir), nprocs=2, join=True)
    got = torch.load(os.path.join(out_dir, "pp_losses.pt"), weights_only=False)
    torch.manual_seed(0)
    ref = _build("qwen3")
    init_normal_(ref, 0.05)
    store = ParamStore(ref, dp_group=None, compute_dtype=torch.float32, device=torch.device("cpu"))
    opt = ShardedAdamW(store, lr=1e-2, weight_decay=0.0)
    mbs, want = _microbatches(), []
    for _ in range(3):
        loss = _loss([ref(**mb)["hidden_states"] for mb in mbs], mbs)
        loss.backward()
        want.append(float(loss.detach()))
        store.finish_backward()
        opt.step()
        opt.zero_grad()
    assert want[2] < want[0]
    assert got == pytest.approx(want, abs=1e-4), (got, want)
