"""Failure detection without any GPU fault: a rank that dies on the host between steps is noticed
by the others through heartbeats (before their next collective) or through a short process-group
timeout; a restarted job resumes from the newest complete checkpoint."""
import os
import socket
import sys
import tempfile
import time
from datetime import timedelta

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _hb_worker(rank, world, port, out_dir):
    from lset_b200.dist.health import PeerFailure, RankHeartbeat

    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    hb = RankHeartbeat(store, rank, world, interval_s=0.1, stale_s=1.0)
    hb.start()
    time.sleep(0.5)
    hb.check_peers()  # everybody alive
    if rank == 1:
        hb.stop()      # this rank "fails" on the host: no more heartbeats, no more steps
        time.sleep(3.0)
        return
    seen = None
    t0 = time.time()
    while time.time() - t0 < 6.0:
        try:
            hb.check_peers()
        except PeerFailure as exc:
            seen = str(exc)
            break
        time.sleep(0.2)
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as fh:
        fh.write(seen or "")
    hb.stop()
    time.sleep(1.0)


def test_heartbeat_detects_dead_peer_between_steps():
    out = tempfile.mkdtemp()
    mp.spawn(_hb_worker, args=(2, _port(), out), nprocs=2, join=True)
    msg = open(os.path.join(out, "r0.txt")).read()
    assert "no heartbeat from rank(s) [1]" in msg


def _pg_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    t = torch.ones(1)
    dist.all_reduce(t)
    if rank == 1:
        os._exit(0)  # leaves between steps, nothing in flight
    err = ""
    try:
        dist.all_reduce(t)  # peer is gone: must end with an error, not hang
    except Exception as exc:
        err = type(exc).__name__
    with open(os.path.join(out_dir, "pg.txt"), "w") as fh:
        fh.write(err)
    os._exit(0)


def test_collective_with_dead_peer_errors_out():
    out = tempfile.mkdtemp()
    t0 = time.time()
    mp.spawn(_pg_worker, args=(2, _port(), out), nprocs=2, join=True)
    assert open(os.path.join(out, "pg.txt")).read() != ""
    assert time.time() - t0 < 60


def test_auto_resume_picks_newest_complete_checkpoint(tmp_path):
    from lset_b200.train.checkpoint import latest_checkpoint

    for step, complete in ((10, True), (20, True), (30, False)):
        d = tmp_path / f"step_{step}"
        d.mkdir()
        if complete:
            torch.save({"step": step}, d / "meta.pt")
    assert latest_checkpoint(str(tmp_path)).endswith("step_20")
    assert latest_checkpoint(str(tmp_path / "missing")) is None


def test_watchdog_exit_code_for_launcher():
    import subprocess

    code = ("import time,sys; sys.path.insert(0,'.');"
            "from lset_b200.train.watchdog import StepWatchdog;"
            "w=StepWatchdog(0.3,poll_s=0.05); w.start(); time.sleep(5)")
    r = subprocess.run([sys.executable, "-c", code], cwd=os.path.dirname(os.path.dirname(__file__)),
                       capture_output=True, text=True, timeout=30)
    assert r.returncode == 75 and "watchdog" in r.stderr


def test_watchdog_gives_a_slow_save_its_own_limit():
    """A phase that is known to be slow (a checkpoint save) runs under an extended idle limit; the
    step limit applies again afterwards."""
    import time

    from lset_b200.train.watchdog import StepWatchdog

    fired = []
    wd = StepWatchdog(0.2, on_timeout=fired.append, poll_s=0.02, exit_process=False)
    wd.start()
    try:
        with wd.extended(5.0):
            time.sleep(0.5)            # two and a half step limits: a slow save
        assert not fired and wd.limit_s == 0.2
        time.sleep(0.1)
        assert not fired               # the clock restarted when the save ended
        time.sleep(0.4)
        assert fired                   # and the step limit is back in force
    finally:
        wd.stop()
