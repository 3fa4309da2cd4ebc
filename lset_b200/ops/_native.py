"""Loader for the native sm_100a library (``lset_b200/_C.so``) and shared call helpers.

The library exports plain C launchers; they are called through ``ctypes`` with raw device pointers
and the current CUDA stream. On a machine with a GPU a missing library is an error (no silent
fallback to eager PyTorch); on a CPU-only machine ``available()`` is False and the ops use their
eager oracle.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "_C.so"
_lib = None
_lock = threading.Lock()
_launches = 0  # number of native kernel launchers called (for benchmark reporting)

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class NativeError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Return the ``ctypes.CDLL`` for the native library. The library in the tree is used when it
    was built from the present sources (a digest stored next to it says so); otherwise it is
    rebuilt first, under a file lock so that the ranks of one job do not build at the same time.
    ``LSET_B200_NO_BUILD=1`` forbids building: a missing or outdated library is then an error."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            from lset_b200.csrc import build as _build

            if not _build.is_current():
                if os.environ.get("LSET_B200_NO_BUILD"):
                    raise NativeError(f"{_LIB_PATH} is missing or older than its sources and "
                                      f"LSET_B200_NO_BUILD is set")
                _build.ensure_built()
            _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


def available() -> bool:
    """True when kernels can run: a CUDA device is visible (the library is then required)."""
    return torch.cuda.is_available()


def use_native(*tensors) -> bool:
    """Native path is taken for CUDA tensors; anything on the CPU goes to the eager oracle."""
    return all(t is None or t.is_cuda for t in tensors) and any(t is not None for t in tensors)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_ptr() -> int:
    """Raw handle of the current CUDA stream of the current device (the C-level lookup: this is
    called once per kernel launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


_status = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write their status code into."""
    t = _status.get(device)          # hot path: the same torch.device object / value every call
    if t is not None:
        return t
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = t
    if device is not None:
        _status[device] = t
    return t


STATUS_NAMES = {
    0: "ok",
    1: "timeout in TMA producer",
    2: "timeout in MMA issuer",
    3: "timeout in epilogue",
    4: "timeout waiting for a peer",
    5: "bad shape",
}


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises when a kernel reported a bounded-wait failure."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise NativeError(f"native kernel reported status {code}: {STATUS_NAMES.get(code, '?')}")


_polls = {}


def poll_status(device=None) -> None:
    """Non-blocking variant of ``check_status`` for the training loop: starts an asynchronous copy
    of the status word into pinned host memory and looks at the copy started by the *previous*
    call (waiting for that old copy costs nothing in steady state). A bounded-wait failure
    therefore raises one or two steps after it happened instead of going unnoticed."""
    word = status_word(device)
    key = (word.device.type, word.device.index)
    prev = _polls.get(key)
    if prev is not None:
        host, event = prev
        event.synchronize()
        code = int(host[0])
        if code != 0:
            word.zero_()
            _polls.pop(key, None)
            raise NativeError(f"native kernel reported status {code}: {STATUS_NAMES.get(code, '?')}")
    else:
        host = torch.zeros(1, dtype=torch.int32).pin_memory()
    host.copy_(word, non_blocking=True)
    event = torch.cuda.Event()
    event.record()
    _polls[key] = (host, event)


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launches() -> int:
    return _launches


def reset_launches() -> None:
    global _launches
    _launches = 0


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")
