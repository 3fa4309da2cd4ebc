"""Symmetric memory: buffers of identical size on every rank of a group, with every peer's copy
mapped into this process, for kernels that read or write other GPUs directly over NVLink.

Allocation and handle exchange go through ``torch.distributed._symmetric_memory`` (the plumbing);
what is returned to the kernels is just the list of peer base pointers. ``enabled()`` reports
whether the runtime should use the peer-memory kernels: CUDA, more than one rank, and
``LSET_B200_SYMM`` not set to ``0``.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist


def enabled(world: int, device: torch.device) -> bool:
    return (world > 1 and device.type == "cuda" and os.environ.get("LSET_B200_SYMM", "1") != "0")


class SymmBuffer:
    """A 1-D symmetric tensor. ``local`` is this rank's copy; ``peer_ptrs[r]`` is rank r's base
    address as seen from this process (``peer_ptrs[rank] == local.data_ptr()``)."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.local = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.local, group)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        # buffer_ptrs are the bases of the peers' symmetric blocks; this tensor may sit at an offset
        off = int(getattr(self.handle, "offset", 0) or 0)
        self.peer_ptrs: List[int] = [int(p) + off for p in self.handle.buffer_ptrs]
        if self.peer_ptrs[self.rank] != self.local.data_ptr():
            raise RuntimeError("symmetric memory: own peer pointer does not match the local tensor "
                               f"({self.peer_ptrs[self.rank]:#x} vs {self.local.data_ptr():#x})")
        self._c_ptrs = (ctypes.c_void_p * self.world)(*self.peer_ptrs)
        self.local.zero_()

    def c_ptr_array(self):
        """``void* const*`` argument for the native launchers (host array of peer pointers)."""
        return self._c_ptrs

    def offset_ptrs(self, byte_offset: int):
        return (ctypes.c_void_p * self.world)(*[p + byte_offset for p in self.peer_ptrs])


def try_alloc(numel: int, dtype, device, group=None) -> Optional[SymmBuffer]:
    """SymmBuffer, or None with a one-line notice when peer mapping is unavailable on this system."""
    try:
        return SymmBuffer(numel, dtype, device, group)
    except Exception as exc:  # pragma: no cover - depends on the machine
        if not getattr(try_alloc, "_warned", False):
            print(f"[lset_b200] symmetric memory unavailable ({type(exc).__name__}: {exc}); "
                  "using NCCL collectives for the sharded runtime", flush=True)
            try_alloc._warned = True
        return None


class DeviceBarrier:
    """Orders the ranks of a group on the current stream with one tiny kernel per rank
    (``lb_device_barrier``: flags in symmetric memory, bounded wait, status word) instead of a
    collective-library call: about a tenth of the host cost of a one-element all-reduce, which
    matters for ops that need one ordering point each (fused tensor-parallel GEMMs, the cross-rank
    loss). ``LSET_B200_DEVICE_BARRIER=0`` falls back to the all-reduce."""

    def __init__(self, device: torch.device, group=None, limit_s: Optional[float] = None):
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        # Ranks reach a barrier at different times (host-side skew of the first steps, allocator
        # stalls); the wait is bounded all the same: 5 s at most (the kernel accepts no more).
        if limit_s is None:
            limit_s = float(os.environ.get("LSET_B200_BARRIER_TIMEOUT_S", "5"))
        self.limit_ns = int(min(max(limit_s, 0.001), 5.0) * 1e9)
        self.epoch = 0
        self.pad = None
        self._token = None
        if os.environ.get("LSET_B200_DEVICE_BARRIER", "1") != "0" and enabled(
                dist.get_world_size(self.group), self.device):
            self.pad = try_alloc(64, torch.int32, self.device, self.group)
            if self.pad is not None:
                # the pads must be zero everywhere before anyone announces epoch 1
                torch.cuda.current_stream(self.device).synchronize()
                dist.barrier(group=self.group)

    def sync(self) -> None:
        if self.pad is None:
            if self._token is None:
                self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
            dist.all_reduce(self._token, group=self.group)
            return
        from ..ops import _native as nv

        self.epoch += 1
        rc = nv.load().lb_device_barrier(
            self.pad.c_ptr_array(), nv.c_int(self.pad.world), nv.c_int(self.pad.rank),
            ctypes.c_uint(self.epoch), ctypes.c_ulonglong(self.limit_ns),
            nv.c_void_p(nv.status_word(self.device).data_ptr()), nv.c_void_p(nv.stream_ptr()))
        nv.check_rc(rc, "lb_device_barrier")
        nv.count_launch()
