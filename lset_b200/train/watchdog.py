"""Host-side failure detection: a step watchdog.

The training loop calls ``beat()`` once per step. A daemon thread checks the time since the last
beat; when it exceeds the limit (a hung collective, a dead peer, a stuck data loader) it prints a
diagnostic, runs the optional ``on_timeout`` callback and ends the process with a non-zero exit
code, so that the launcher (``torchrun --max-restarts``) can restart the job, which then resumes
from the newest complete checkpoint. The reference has no counterpart (no watchdog, heartbeat or
timeout anywhere; lset/cli.py:56-67 only propagates the launcher's return code).
"""
from __future__ import annotations

import os
import sys
import threading
import time
from typing import Callable, Optional

EXIT_CODE = 75  # EX_TEMPFAIL: the job may be retried


class StepWatchdog:
    def __init__(self, limit_s: float, on_timeout: Optional[Callable[[float], None]] = None,
                 poll_s: Optional[float] = None, exit_process: bool = True):
        self.limit_s = float(limit_s)
        self.on_timeout = on_timeout
        self.poll_s = poll_s if poll_s is not None else max(0.05, min(1.0, self.limit_s / 4))
        self.exit_process = exit_process
        self.fired = False
        self._last = time.monotonic()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def beat(self) -> None:
        self._last = time.monotonic()

    def extended(self, limit_s: float):
        """Context manager for a phase that legitimately takes longer than a step (writing a
        checkpoint, loading one): inside it the idle limit is ``limit_s``; the clock restarts on
        entry and on exit."""
        import contextlib

        @contextlib.contextmanager
        def scope():
            prev = self.limit_s
            self.limit_s = max(float(limit_s), prev)
            self.beat()
            try:
                yield
            finally:
                self.beat()
                self.limit_s = prev

        return scope()

    def start(self) -> None:
        if self._thread is not None:
            return
        self.beat()
        self._thread = threading.Thread(target=self._run, name="lset-b200-watchdog", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.poll_s + 1)
            self._thread = None

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            idle = time.monotonic() - self._last
            if idle > self.limit_s:
                self.fired = True
                rank = os.environ.get("RANK", "0")
                print(f"[watchdog] rank {rank}: no training step finished for {idle:.1f} s "
                      f"(limit {self.limit_s:.1f} s); aborting", file=sys.stderr, flush=True)
                if self.on_timeout is not None:
                    try:
                        self.on_timeout(idle)
                    except Exception as exc:  # pragma: no cover
                        print(f"[watchdog] on_timeout raised {exc!r}", file=sys.stderr)
                if self.exit_process:
                    os._exit(EXIT_CODE)
                return


class InjectedFailure(RuntimeError):
    """Raised by ``maybe_fail`` (host-side fault injection)."""


def maybe_fail(step: int, rank: int) -> None:
    """Host-side fault injection for recovery tests and drills.

    ``LSET_B200_FAIL_AT_STEP="<step>[,<rank>[,<mode>]]"`` makes rank ``<rank>`` (default 0) fail
    right before optimizer step ``<step>`` on the first attempt of a job (a group restarted by the
    launcher runs through): ``mode`` ``raise`` (default) raises ``InjectedFailure``, ``exit`` ends
    the process with the watchdog's exit code, ``hang`` sleeps on the host (what a stuck data
    loader looks like; the step watchdog is what ends it). The failure happens between steps on the host; on a
    GPU the device is synchronised first, so no kernel or collective of this rank is in flight.
    Nothing on the device is made to fault.
    """
    spec = os.environ.get("LSET_B200_FAIL_AT_STEP")
    if not spec or int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")) > 0:
        return
    parts = spec.split(",")
    if step != int(parts[0]) or rank != (int(parts[1]) if len(parts) > 1 and parts[1] else 0):
        return
    try:
        import torch

        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.synchronize()
    except Exception:  # pragma: no cover - best effort before leaving
        pass
    mode = parts[2] if len(parts) > 2 else "raise"
    print(f"[fault injection] rank {rank} fails before step {step} ({mode})", file=sys.stderr, flush=True)
    if mode == "exit":
        os._exit(EXIT_CODE)
    if mode == "hang":
        while True:
            time.sleep(3600.0)
    raise InjectedFailure(f"injected failure on rank {rank} before step {step}")
