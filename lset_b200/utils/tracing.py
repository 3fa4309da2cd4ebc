"""Tracing and timing helpers (the reference has none: no profiler hooks, NVTX ranges or timers).

* ``nvtx_range(name)``: NVTX range when CUDA is available, no-op otherwise.
* ``PhaseTimer``: device-side time per named phase with CUDA events on the current stream; totals
  are read with one synchronisation at report time and can be max-reduced over ranks.
* ``roofline(...)``: achieved fraction of the measured peaks (``MEASURED_PEAKS.json`` format:
  ``hbm_gbs``, ``bf16_tflops``, ``bf16_tflops_sustained``) for a kernel's bytes / FLOPs / time.
"""
from __future__ import annotations

import contextlib
import json
import os
from collections import defaultdict
from typing import Dict, Optional

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer copy on this class of machine (900 nominal)


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._pairs = defaultdict(list)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        with nvtx_range(name):
            yield
        b.record()
        self._pairs[name].append((a, b))

    def report(self, reduce_max_group=None, reset: bool = True) -> Dict[str, float]:
        """Milliseconds per phase (sum over recorded intervals); max over ranks when a process
        group (or ``True`` for the default group) is given."""
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        out = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self._pairs.items()}
        if reduce_max_group is not None and torch.distributed.is_initialized():
            keys = sorted(out)
            t = torch.tensor([out[k] for k in keys], device="cuda")
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX,
                                         group=None if reduce_max_group is True else reduce_max_group)
            out = dict(zip(keys, t.tolist()))
        if reset:
            self._pairs.clear()
        return out


def load_peaks(path: Optional[str] = None) -> dict:
    """Measured peaks, or the documented fallback values when the file is absent."""
    cand = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(cand) as fh:
            d = json.load(fh)
        return dict(FALLBACK_PEAKS, **{k: d[k] for k in FALLBACK_PEAKS if k in d}, source="measured")
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


def roofline(ms: float, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0,
             peaks: Optional[dict] = None, sustained: bool = False) -> dict:
    """Achieved rates and the fraction of the binding roof for one kernel or fused path."""
    p = peaks or load_peaks()
    t = ms / 1e3
    peak_tf = p["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    floors = {"compute": flops / (peak_tf * 1e12), "hbm": hbm_bytes / (p["hbm_gbs"] * 1e9),
              "nvlink": nvlink_bytes / (NVLINK_GBS_PER_DIRECTION * 1e9)}
    bound = max(floors, key=floors.get)
    return {"tflops": flops / t / 1e12 if t else 0.0, "hbm_gbs": hbm_bytes / t / 1e9 if t else 0.0,
            "nvlink_gbs": nvlink_bytes / t / 1e9 if t else 0.0, "bound": bound,
            "fraction_of_roof": floors[bound] / t if t else 0.0, "peaks": p.get("source")}
