"""Snapshot of the CPU and CUDA random state, restorable inside a ``with`` block, so the dropout
masks of the no-grad embedding pass and of the gradient replay agree
(cf. lset/train/grad_cache/rand_context.py:11-27)."""
from __future__ import annotations

import torch


class RandContext:
    def __init__(self, *tensors):
        self.cpu_state = torch.get_rng_state()
        devs = sorted({t.device.index for t in tensors
                       if torch.is_tensor(t) and t.is_cuda and t.device.index is not None})
        self.devices = devs
        self.cuda_states = [torch.cuda.get_rng_state(d) for d in devs]
        self._fork = None

    def __enter__(self):
        self._fork = torch.random.fork_rng(devices=self.devices)
        self._fork.__enter__()
        torch.set_rng_state(self.cpu_state)
        for d, s in zip(self.devices, self.cuda_states):
            torch.cuda.set_rng_state(s, d)
        return self

    def __exit__(self, *exc):
        fork, self._fork = self._fork, None
        return fork.__exit__(*exc)
