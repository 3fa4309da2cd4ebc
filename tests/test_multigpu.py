"""Multi-GPU checks (skipped with fewer than two GPUs): the peer-memory sharded path (fused
reduce-scatter + norm, fused AdamW + push all-gather) must match the NCCL path."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, symm, tmp_path, port):
    out = tmp_path / f"r_{symm}.json"
    env = dict(os.environ, LSET_B200_SYMM=str(symm), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "mgpu_worker.py"), str(out), "3"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return json.loads(out.read_text())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_symm_path_matches_nccl_path(tmp_path):
    world = 2
    a = _run(world, 0, tmp_path, 29631)
    b = _run(world, 1, tmp_path, 29632)
    assert a["symm"] is False and b["symm"] is True
    assert a["replicas_equal"] and b["replicas_equal"]
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 5e-2 * max(1.0, abs(x)), (a["losses"], b["losses"])
    for x, y in zip(a["norms"], b["norms"]):
        assert abs(x - y) < 2e-2 * max(1.0, abs(x)), (a["norms"], b["norms"])
    for x, y in zip(a["sumsq"], b["sumsq"]):
        assert abs(x - y) < 1e-3 * max(1.0, abs(x)), (a["sumsq"], b["sumsq"])


def _run_loss(world, tmp_path, port):
    out = tmp_path / "loss.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "mgpu_loss_worker.py"), str(out)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return json.loads(out.read_text())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_cross_rank_infonce_matches_gather_path(tmp_path):
    r = _run_loss(2, tmp_path, 29641)
    for case in r["cases"]:
        assert case["loss_err"] < 2e-2, case
        assert case["dq_err"] < 3e-2 and case["dk_err"] < 3e-2, case


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_sequence_parallel_tp(tmp_path):
    """All-gather fused into the GEMM, reduce-scatter fused into its epilogue, and a
    sequence-parallel decoder built on both, against plain PyTorch."""
    out = tmp_path / "tp.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29651",
           os.path.join(HERE, "mgpu_tp_worker.py"), str(out)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    r = json.loads(out.read_text())
    assert r["fused"] and r["model"]["sp_fused"], "peer-memory path not active on this box"
    for case in r["cases"]:
        for k in ("y", "dx", "dw", "db"):
            if k in case:
                assert case[k] < 2e-2, case
    assert r["model"]["hidden"] < 5e-2 and r["model"]["worst_grad"] < 5e-2, r["model"]
