"""Sharded data parallelism (ZeRO) over flat parameter groups, and the AdamW that runs on it.

This is the framework's counterpart of the reference's FSDP2 set-up
(lset/distributed/parallel.py:129-160: one group per transformer layer plus a root group, bf16
compute parameters, fp32 gradient reduction and fp32 optimizer state) built for B200 memory sizes:

* every group owns one flat **bf16** buffer holding its trainable parameters (the tensors the
  kernels read), one flat **fp32 gradient accumulator** (``param.main_grad`` views; weight-gradient
  GEMMs add straight into it, so gradient accumulation and the bf16->fp32 cast cost nothing), and,
  for the 1/W slice this rank owns, fp32 master weights and AdamW moments;
* backward: as soon as a layer's backward has run, its gradient buffer is reduce-scattered (fp32,
  averaged) on a side stream, overlapping the rest of backward; with gradient accumulation the
  reduction only happens on the boundary micro-step;
* step: global-norm clipping with the coefficient kept on the device, one fused AdamW kernel per
  group that also writes the new bf16 shard, then an all-gather of the shards that the next
  forward waits for per layer. With 180 GB per GPU the bf16 replica stays resident by default (no
  re-gather in backward).
* ``reshard_after_forward=True`` selects the parameter-sharded mode (ZeRO-3, what the reference's
  ``fully_shard`` does per layer, lset/distributed/parallel.py:129-160): a layer group keeps only
  its 1/W bf16 shard; the full parameters of a layer live in one of two rotating buffers, gathered
  (peer loads over NVLink, or NCCL) on the side stream one layer ahead of the forward and again one
  layer ahead of the backward; the layer's fp32 gradients are written into one of two rotating
  buffers and reduced into the 1/W gradient shard as soon as its backward is done. Parameter,
  gradient and optimizer memory of the layers then fall with the data-parallel size. The root
  group (embeddings, final norm) stays resident.

Collectives go through ``torch.distributed`` (NCCL on GPUs, gloo on CPU for tests) unless the
symmetric-memory kernels of ``lset_b200.dist.symm`` are enabled, which fuse the gradient
reduce-scatter, the optimizer step and the parameter all-gather into two launches over NVLink.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _native as nv
from ..ops._grads import register_main_grad
from ..ops.norm import scratch

_ALIGN = 8  # elements; keeps every parameter 16-byte aligned in the bf16 buffer


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatGroup:
    """One communication / optimizer unit: the trainable parameters of a set of modules."""

    def __init__(self, name: str, params: Sequence[nn.Parameter], world: int, rank: int,
                 compute_dtype: torch.dtype, device: torch.device, group=None, use_symm: bool = False,
                 shard_params: bool = False):
        self.name = name
        # parameter-sharded mode: only the 1/W slice of parameters and gradients is kept here; the
        # store binds the parameters to a rotating full buffer while the layer runs
        self.sharded = bool(shard_params) and world > 1
        self.pslot = self.gslot = None
        self.has_grad = False
        self.params = list(params)
        self.world, self.rank = world, rank
        offs, n = [], 0
        for p in self.params:
            offs.append(n)
            n += _round_up(p.numel(), _ALIGN)
        self.offsets = offs
        self.numel = _round_up(max(n, _ALIGN), _ALIGN * world)
        self.shard_numel = self.numel // world
        self.lo = rank * self.shard_numel
        self.hi = self.lo + self.shard_numel
        self.device = device
        self.compute_dtype = compute_dtype
        # master values come from the parameters as given (fp32 when the module was built in fp32)
        full_master = torch.zeros(self.numel, dtype=torch.float32, device=device)
        for p, o in zip(self.params, offs):
            full_master[o:o + p.numel()] = p.data.detach().reshape(-1).to(device, torch.float32)
        self.symm_param = self.symm_grad = self.symm_shard = None
        if self.sharded:
            if use_symm and compute_dtype == torch.bfloat16:
                from . import symm

                self.symm_shard = symm.try_alloc(self.shard_numel, compute_dtype, device, group)
            self.param_shard = (self.symm_shard.local if self.symm_shard is not None else
                                torch.empty(self.shard_numel, dtype=compute_dtype, device=device))
            self.param_shard.copy_(full_master[self.lo:self.hi].to(compute_dtype))
            self.flat_param = self.flat_grad = None
            self.master = full_master[self.lo:self.hi].clone()
            del full_master
            self.exp_avg = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
            self.exp_avg_sq = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
            self.grad_shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
            self.reduce_event = self.gather_event = None
            self.reduced = False
            return
        if use_symm and compute_dtype == torch.bfloat16:
            from . import symm

            self.symm_param = symm.try_alloc(self.numel, compute_dtype, device, group)
            self.symm_grad = (symm.try_alloc(self.numel, torch.float32, device, group)
                              if self.symm_param is not None else None)
        if self.symm_grad is not None:
            self.flat_param = self.symm_param.local
            self.flat_param.copy_(full_master.to(compute_dtype))
            self.flat_grad = self.symm_grad.local
        else:
            self.symm_param = None
            self.flat_param = full_master.to(compute_dtype)
            self.flat_grad = torch.zeros(self.numel, dtype=torch.float32, device=device)
        self.master = full_master[self.lo:self.hi].clone()
        del full_master
        self.exp_avg = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        self.exp_avg_sq = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        self.grad_shard = (self.flat_grad if world == 1 else
                           torch.zeros(self.shard_numel, dtype=torch.float32, device=device))
        for p, o in zip(self.params, offs):
            p.data = self.flat_param[o:o + p.numel()].view(p.shape)
            p.main_grad = self.flat_grad[o:o + p.numel()].view(p.shape)
            register_main_grad(p)   # found by storage address too (detached aliases under AC)
            p.grad = None
        self.reduce_event = None     # recorded after the gradient reduction of this group
        self.gather_event = None     # recorded after the parameter all-gather of this group
        self.reduced = False

    def collect_autograd_grads(self) -> None:
        """Fold any ``param.grad`` that autograd produced (ops without main_grad support) into the
        fp32 accumulator."""
        for p in self.params:
            if p.grad is not None:
                if getattr(p, "main_grad", None) is not None:
                    p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None

    def bind_params(self, buf: torch.Tensor) -> None:
        """Point the parameters at their places in a full bf16 buffer."""
        for p, o in zip(self.params, self.offsets):
            n = p.numel()
            p.data = buf[o:o + n].view(p.shape)

    def bind_grads(self, buf: torch.Tensor) -> None:
        for p, o in zip(self.params, self.offsets):
            n = p.numel()
            p.main_grad = buf[o:o + n].view(p.shape)
            register_main_grad(p)


class ParamStore:
    """Flat, sharded storage for a module's trainable parameters."""

    def __init__(self, module: nn.Module, layer_modules: Optional[Iterable[nn.Module]] = None,
                 dp_group=None, compute_dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, reshard_after_forward: bool = False,
                 overlap: bool = True, tp_group=None):
        self.module = module
        self.dp_group = dp_group
        self.tp_group = tp_group
        if dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(dp_group), dist.get_rank(dp_group)
        else:
            self.world, self.rank = 1, 0
        if device is None:
            device = next(module.parameters()).device
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        self.requires_gradient_sync = True
        from . import symm as _symm

        self.use_symm = _symm.enabled(self.world, self.device)
        self.tp_world = dist.get_world_size(tp_group) if tp_group is not None else 1
        # parameter-sharded mode: layer groups only, every parameter trainable (module backward
        # hooks drive the gathers; a frozen first layer would not fire them), no tensor parallelism
        frozen = any(not p.requires_grad for p in module.parameters())
        self.zero3 = bool(reshard_after_forward) and self.world > 1 and self.tp_world == 1 and not frozen
        if reshard_after_forward and self.world > 1 and not self.zero3:
            print("[lset_b200] reshard_after_forward needs tp_size == 1 and no frozen parameters; "
                  "keeping the resident-replica mode", flush=True)
        self.groups: List[FlatGroup] = []
        claimed = set()
        layers = list(layer_modules) if layer_modules is not None else list(getattr(module, "layers", []))
        self._groups_of_layer = []  # (layer module, [groups])

        def make_groups(name, ps):
            # tensor-parallel shards and replicated parameters go to separate groups: their
            # squared norms are combined differently across the tensor-parallel ranks
            out = []
            def kind(p):
                if getattr(p, "_tp_sharded", False):
                    return ".tp"
                return ".tpp" if getattr(p, "_tp_partial_grad", False) else ""

            for tag in ("", ".tp", ".tpp"):
                sel = [p for p in ps if kind(p) == tag]
                if sel:
                    g = FlatGroup(name + tag, sel, self.world, self.rank, compute_dtype, self.device,
                                  dp_group, self.use_symm,
                                  shard_params=self.zero3 and name != "root")
                    g.tp_sharded = tag == ".tp"
                    # replicated parameter whose per-rank gradient is only a part of the total
                    # (per-head norm weights; everything token-sharded under sequence parallelism)
                    g.tp_partial = tag == ".tpp"
                    out.append(g)
            return out

        for i, layer in enumerate(layers):
            ps = [p for p in layer.parameters() if p.requires_grad and id(p) not in claimed]
            claimed.update(id(p) for p in ps)
            if ps:
                gs = make_groups(f"layers.{i}", ps)
                self._groups_of_layer.append((layer, gs))
                self.groups.extend(gs)
        rest = [p for p in module.parameters() if p.requires_grad and id(p) not in claimed]
        if rest:
            self.groups.extend(make_groups("root", rest))
        self.use_symm = self.use_symm and all(
            (g.symm_shard if g.sharded else g.symm_grad) is not None for g in self.groups)
        # squared norm of the reduced shards: [0] replicated parameters, [1] tensor-parallel shards
        self.sumsq = torch.zeros(2, dtype=torch.float32, device=self.device)
        # frozen parameters and buffers: just move / cast, they stay replicated
        for p in module.parameters():
            if not p.requires_grad:
                p.data = p.data.to(self.device, compute_dtype if p.is_floating_point() else p.dtype)
        for b in module.buffers():
            b.data = b.data.to(self.device)
        self.overlap = overlap and self.device.type == "cuda" and self.world > 1
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.overlap else None
        self._hooks = []
        if self.zero3:
            self._init_pools()
        if self.world > 1 or self.tp_world > 1:
            self._install_hooks()

    # ------------------------------------------------------------------ parameter-sharded mode
    def _init_pools(self) -> None:
        """Two rotating full-size buffers for parameters and two for gradients (the largest layer
        group sets their size). The gradient buffers are read by the peers' reduce kernels, so
        they are symmetric allocations when the peer-memory path is on."""
        sharded = [g for g in self.groups if g.sharded]
        n = max(g.numel for g in sharded)
        self._pbuf = [torch.empty(n, dtype=self.compute_dtype, device=self.device) for _ in range(2)]
        self._pfree = [None, None]       # event after which a parameter buffer may be overwritten
        self._powner = [None, None]      # group whose parameters the buffer holds (valid contents)
        self._gsymm = [None, None]
        if self.use_symm:
            from . import symm as _symm

            self._gsymm = [_symm.try_alloc(n, torch.float32, self.device, self.dp_group)
                           for _ in range(2)]
            if any(b is None for b in self._gsymm):
                self.use_symm = False
        self._gbuf = [b.local if (self.use_symm and b is not None) else
                      torch.zeros(n, dtype=torch.float32, device=self.device) for b in self._gsymm]
        self._gfree = [None, None]
        self._gowner = [None, None]
        self._order = {id(g): i for i, g in enumerate(sharded)}
        self._sharded = sharded
        for g in sharded:                # valid shapes from the start; contents arrive with a gather
            g.bind_params(self._pbuf[0])
            for p in g.params:
                p.main_grad = None
                p.grad = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.dp_group)   # every rank's shards are in place before any gather

    def _stream(self):
        return torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None

    def _materialize(self, g: FlatGroup, wait: bool = True) -> None:
        """Make the full parameters of a sharded group available: reuse a buffer that still holds
        them, or gather the shards of all ranks into a free one on the side stream. ``wait`` makes
        the current stream wait for the gather (a prefetch passes False)."""
        if g.pslot is None:
            slot = next((i for i in range(2) if self._powner[i] is g), None)
            if slot is None:
                busy = {x.pslot for x in self._sharded if x.pslot is not None}
                slot = next((i for i in range(2) if i not in busy), None)
                if slot is None:
                    return                      # both buffers in use: gathered on demand later
                self._gather_into(g, slot)
            g.pslot = slot
            self._powner[slot] = g
            g.bind_params(self._pbuf[slot])
        if wait and g.gather_event is not None:
            torch.cuda.current_stream(self.device).wait_event(g.gather_event)
            g.gather_event = None

    def _gather_into(self, g: FlatGroup, slot: int) -> None:
        dst = self._pbuf[slot][:g.numel]
        cur = self._stream()
        side = self.comm_stream
        if side is not None:
            side.wait_stream(cur)
            if self._pfree[slot] is not None:
                side.wait_event(self._pfree[slot])
        ctx = torch.cuda.stream(side) if side is not None else _null_context()
        with ctx:
            if self.use_symm:
                rc = nv.load().lb_gather_shards(
                    g.symm_shard.c_ptr_array(), nv.c_int(self.world), nv.c_int(self.rank),
                    nv.c_ll(g.shard_numel * g.param_shard.element_size()),
                    nv.c_void_p(dst.data_ptr()), nv.c_void_p(nv.stream_ptr()))
                nv.check_rc(rc, "lb_gather_shards")
                nv.count_launch()
            elif dst.is_cuda:
                dist.all_gather_into_tensor(dst, g.param_shard, group=self.dp_group)
            else:
                parts = [torch.empty_like(g.param_shard) for _ in range(self.world)]
                dist.all_gather(parts, g.param_shard, group=self.dp_group)
                dst.copy_(torch.cat(parts))
            if side is not None:
                g.gather_event = torch.cuda.Event()
                g.gather_event.record(side)
        self._pfree[slot] = None

    def _release_params(self, g: FlatGroup) -> None:
        """The layer is done with its parameters: the buffer may be reused once the work queued so
        far has run (its contents stay valid until then and are reused if nobody took it)."""
        if g.pslot is None:
            return
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._pfree[g.pslot] = ev
        g.pslot = None

    def _acquire_grads(self, g: FlatGroup) -> None:
        """Bind a zeroed full gradient buffer to the group for its backward."""
        if g.gslot is not None:
            return
        busy = {x.gslot for x in self._sharded if x.gslot is not None}
        slot = next((i for i in range(2) if i not in busy), None)
        if slot is None:
            raise RuntimeError("parameter-sharded mode: more than two layers in backward at once")
        if self._gfree[slot] is not None and self.device.type == "cuda":
            torch.cuda.current_stream(self.device).wait_event(self._gfree[slot])
            self._gfree[slot] = None
        buf = self._gbuf[slot][:g.numel]
        buf.zero_()
        g.gslot = slot
        g.reduced = False
        g.bind_grads(buf)

    def _neighbour(self, g: FlatGroup, step: int) -> Optional[FlatGroup]:
        i = self._order[id(g)] + step
        return self._sharded[i] if 0 <= i < len(self._sharded) else None

    # ------------------------------------------------------------------ hooks
    def _install_hooks(self) -> None:
        # Forward passes of a layer that still await their backward. A step may run a layer more
        # than once before one backward call (queries and documents encoded separately on padded
        # batches): a resident group is reduced when the last of those passes has been through
        # backward, not at the first hook that fires.
        self._pending = {}
        # Layers that ran a pass none of whose inputs requires a gradient (the first block behind
        # frozen embeddings: LoRA, QLoRA): torch then fires the module's backward hook when the
        # gradients of its *outputs* are ready, before the layer's own parameters have received
        # theirs. Such a layer is not reduced from the hook; `finish_backward` does it.
        self._fires_early = {}
        for layer, gs in self._groups_of_layer:
            self._pending[id(layer)] = 0
            self._fires_early[id(layer)] = False

            def after_backward(_mod, _gin, _gout, gs=gs, key=id(layer)):
                left = self._pending[key] = max(0, self._pending[key] - 1)
                for g in gs:
                    # sharded groups reduce on every pass and micro-step (their full gradient
                    # buffer is handed on to the next layer); resident ones only on the boundary
                    # step, after the last pass
                    if g.sharded or (self.requires_gradient_sync and left == 0
                                     and not self._fires_early[key]):
                        self._reduce_group(g)
                    if g.sharded:
                        self._release_params(g)

            def before_forward(_mod, _args, gs=gs, key=id(layer)):
                if torch.is_grad_enabled():
                    self._pending[key] += 1
                    if not any(torch.is_tensor(a) and a.requires_grad for a in _args):
                        self._fires_early[key] = True
                for g in gs:
                    if g.sharded:
                        self._materialize(g)
                        nxt = self._neighbour(g, +1)
                        if nxt is not None:
                            self._materialize(nxt, wait=False)   # next layer, one layer ahead
                    else:
                        self._wait_gather(g)

            def after_forward(_mod, _args, _out, gs=gs):
                for g in gs:
                    if g.sharded:
                        self._release_params(g)

            def before_backward(_mod, _gout, gs=gs):
                for g in gs:
                    if g.sharded:
                        self._materialize(g)
                        self._acquire_grads(g)
                        prv = self._neighbour(g, -1)
                        if prv is not None:
                            self._materialize(prv, wait=False)

            self._hooks.append(layer.register_full_backward_hook(after_backward))
            self._hooks.append(layer.register_forward_pre_hook(before_forward))
            if any(g.sharded for g in gs):
                self._hooks.append(layer.register_forward_hook(after_forward))
                self._hooks.append(layer.register_full_backward_pre_hook(before_backward))

    def set_requires_gradient_sync(self, flag: bool) -> None:
        """False on non-boundary micro-steps of gradient accumulation (gradients only accumulate)."""
        self.requires_gradient_sync = bool(flag)

    # ------------------------------------------------------------------ collectives
    def _reduce_group(self, g: FlatGroup) -> None:
        if g.reduced:
            return
        g.collect_autograd_grads()
        if g.sharded:
            self._reduce_sharded(g)
            return
        if getattr(g, "tp_partial", False) and self.tp_world > 1:
            dist.all_reduce(g.flat_grad, op=dist.ReduceOp.SUM, group=self.tp_group)
        if self.world == 1:
            g.reduced = True
            return
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self._reduce_scatter(g)
                g.reduce_event = torch.cuda.Event()
                g.reduce_event.record(self.comm_stream)
        else:
            self._reduce_scatter(g)
        g.reduced = True

    def _reduce_sharded(self, g: FlatGroup) -> None:
        """Reduce the group's full gradient buffer into its 1/W shard (averaged, added to what
        earlier micro-steps left there) and hand the buffer back."""
        if g.gslot is None:
            return
        slot = g.gslot
        buf = self._gbuf[slot][:g.numel]
        side = self.comm_stream
        if side is not None:
            side.wait_stream(torch.cuda.current_stream(self.device))
        ctx = torch.cuda.stream(side) if side is not None else _null_context()
        with ctx:
            if self.use_symm:
                # every rank's buffer complete before anyone reads it; everyone done reading before
                # anyone zeroes it for another layer
                self._barrier("reduce").sync()
                lib = nv.load()
                scr = scratch("reduce_shard", lib.lb_reduce_shard_partial_rows(), self.device)
                rc = lib.lb_reduce_shard_f32(
                    self._gsymm[slot].c_ptr_array(), nv.c_int(self.world), nv.c_int(self.rank),
                    nv.c_ll(g.lo), nv.c_ll(g.shard_numel), nv.c_float(1.0 / self.world),
                    nv.c_void_p(g.grad_shard.data_ptr()), nv.c_void_p(scr.data_ptr()),
                    nv.c_void_p(0), nv.c_int(int(g.has_grad)), nv.c_void_p(nv.stream_ptr()))
                nv.check_rc(rc, "lb_reduce_shard_f32")
                nv.count_launch()
                self._barrier("reduce_done").sync()
            elif buf.is_cuda:
                tmp = torch.empty_like(g.grad_shard)
                dist.reduce_scatter_tensor(tmp, buf, op=dist.ReduceOp.AVG, group=self.dp_group)
                g.grad_shard.add_(tmp) if g.has_grad else g.grad_shard.copy_(tmp)
            else:
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.dp_group)
                part = buf[g.lo:g.hi] / self.world
                g.grad_shard.add_(part) if g.has_grad else g.grad_shard.copy_(part)
            if side is not None:
                ev = torch.cuda.Event()
                ev.record(side)
                g.reduce_event = ev
                self._gfree[slot] = ev
        g.has_grad = True
        g.gslot = None
        g.reduced = True
        for p in g.params:
            p.main_grad = None

    def _reduce_scatter(self, g: FlatGroup) -> None:
        if self.use_symm:
            # All ranks' gradients for this group must be complete before anyone reads them: a
            # device barrier on this (side) stream orders the kernels across ranks.
            self._barrier("reduce").sync()
            lib = nv.load()
            scr = scratch("reduce_shard", lib.lb_reduce_shard_partial_rows(), self.device)
            rc = lib.lb_reduce_shard_f32(
                g.symm_grad.c_ptr_array(), nv.c_int(self.world), nv.c_int(self.rank), nv.c_ll(g.lo),
                nv.c_ll(g.shard_numel), nv.c_float(1.0 / self.world),
                nv.c_void_p(g.grad_shard.data_ptr()), nv.c_void_p(scr.data_ptr()),
                nv.c_void_p(0 if self.zero3 else
                            self.sumsq.data_ptr() + (4 if getattr(g, "tp_sharded", False) else 0)),
                nv.c_int(0), nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_reduce_shard_f32")
            nv.count_launch(1 if self.zero3 else 2)
            return
        if g.flat_grad.is_cuda:
            dist.reduce_scatter_tensor(g.grad_shard, g.flat_grad, op=dist.ReduceOp.AVG,
                                       group=self.dp_group)
        else:  # gloo: no reduce-scatter
            dist.all_reduce(g.flat_grad, op=dist.ReduceOp.SUM, group=self.dp_group)
            g.grad_shard.copy_(g.flat_grad[g.lo:g.hi]).div_(self.world)

    def _barrier(self, name: str):
        """Device barrier (flags in symmetric memory) per use site: the sites run on different
        streams, so each keeps its own epoch sequence."""
        bars = self.__dict__.setdefault("_barriers", {})
        if name not in bars:
            from . import symm as _symm

            bars[name] = _symm.DeviceBarrier(self.device, self.dp_group)
        return bars[name]

    def _token(self) -> torch.Tensor:
        if getattr(self, "_tok", None) is None:
            self._tok = torch.zeros(1, dtype=torch.float32, device=self.device)
        return self._tok

    def finish_backward(self) -> None:
        """Call after ``loss.backward()``: reduces whatever the hooks did not cover (root group,
        layers whose inputs carry no gradient) and folds stray autograd grads in."""
        for g in self.groups:
            g.collect_autograd_grads()
        for key in getattr(self, "_pending", ()):
            self._pending[key] = 0          # passes that never reached backward do not carry over
        if not self.requires_gradient_sync:
            return
        for g in reversed(self.groups):
            if g.sharded:
                if g.gslot is not None:       # backward reached the layer but not its input
                    self._reduce_group(g)
                    self._release_params(g)
                continue
            if not g.reduced:
                self._reduce_group(g)
        for key in getattr(self, "_fires_early", ()):
            self._fires_early[key] = False

    def wait_reductions(self) -> None:
        for g in self.groups:
            if g.reduce_event is not None:
                torch.cuda.current_stream().wait_event(g.reduce_event)
                g.reduce_event = None

    def gather_params(self) -> None:
        """All-gather the updated bf16 shards (after an optimizer step)."""
        if self.world == 1:
            return
        if self.zero3:
            self._powner = [None, None]     # the gathered copies are stale now
        if self.use_symm:
            # adamw_push already stored the new shards into every rank's buffer; one barrier
            # orders "all pushes done" (and, in the parameter-sharded mode, "all shards updated")
            # before the next forward on every rank.
            self._barrier("gather").sync()
            return
        hooked = {id(g) for _, gs in self._groups_of_layer for g in gs}
        for g in self.groups:
            if g.sharded:
                continue                    # gathered layer by layer in the next forward
            if self.comm_stream is not None:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream):
                    dist.all_gather_into_tensor(g.flat_param, g.flat_param[g.lo:g.hi],
                                                group=self.dp_group)
                    g.gather_event = torch.cuda.Event()
                    g.gather_event.record(self.comm_stream)
            else:
                dist.all_gather_into_tensor(g.flat_param, g.flat_param[g.lo:g.hi].clone(),
                                            group=self.dp_group)
        # Groups that belong to a layer are waited for by that layer's forward hook. The others
        # (embeddings, final norm, a task's own parameters) have no hook and are read first by the
        # next forward: the compute stream waits for them here.
        for g in self.groups:
            if id(g) not in hooked:
                self._wait_gather(g)

    def _wait_gather(self, g: FlatGroup) -> None:
        if g.gather_event is not None:
            torch.cuda.current_stream().wait_event(g.gather_event)
            g.gather_event = None

    def wait_all_gathers(self) -> None:
        for g in self.groups:
            self._wait_gather(g)

    # ------------------------------------------------------------------ utilities
    def zero_grad(self) -> None:
        for g in self.groups:
            if g.sharded:
                g.has_grad = False          # the next reduction overwrites the shard
            else:
                g.flat_grad.zero_()
            g.reduced = False
        self.sumsq.zero_()

    def memory_report(self) -> dict:
        """Bytes this rank holds for trainable parameters, gradients and optimizer state."""
        nb = lambda t: t.numel() * t.element_size()  # noqa: E731
        rep = {"param_bytes": 0, "grad_bytes": 0, "optim_bytes": 0, "pool_bytes": 0,
               "sharded_groups": sum(1 for g in self.groups if g.sharded), "world": self.world}
        for g in self.groups:
            rep["param_bytes"] += nb(g.param_shard) if g.sharded else nb(g.flat_param)
            if not g.sharded:
                rep["grad_bytes"] += nb(g.flat_grad)
            if g.sharded or g.grad_shard is not g.flat_grad:
                rep["grad_bytes"] += nb(g.grad_shard)
            rep["optim_bytes"] += nb(g.master) + nb(g.exp_avg) + nb(g.exp_avg_sq)
        if self.zero3:
            rep["pool_bytes"] = sum(nb(b) for b in self._pbuf) + sum(nb(b) for b in self._gbuf)
        return rep

    def trainable_parameters(self):
        for g in self.groups:
            yield from g.params

    def canonical_index(self) -> dict:
        """``id(param) -> position`` among the module's trainable parameters in module order: the
        numbering of ``torch.optim`` state dicts, independent of how this store grouped them."""
        hit = self.__dict__.get("_canon")
        if hit is None:
            owned = {id(p) for p in self.trainable_parameters()}
            hit, n = {}, 0
            for p in self.module.parameters():
                if id(p) in owned and id(p) not in hit:
                    hit[id(p)] = n
                    n += 1
            self._canon = hit
        return hit

    def named_master_tensors(self):
        """``(name, fp32 tensor)`` for every trainable parameter, gathered across ranks (a
        collective when world > 1). Used for checkpoints."""
        names = {id(p): n for n, p in self.module.named_parameters()}
        for g in self.groups:
            full = self._gather_fp32(g, g.master)
            for p, o in zip(g.params, g.offsets):
                yield names[id(p)], full[o:o + p.numel()].view(p.shape)

    def _gather_fp32(self, g: FlatGroup, shard: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return shard
        full = torch.empty(g.numel, dtype=torch.float32, device=shard.device)
        if shard.is_cuda:
            dist.all_gather_into_tensor(full, shard.contiguous(), group=self.dp_group)
        else:
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard.contiguous(), group=self.dp_group)
            full = torch.cat(parts)
        return full

    def load_master(self, name_to_tensor: dict) -> None:
        """Overwrite master weights and bf16 parameters from full tensors keyed by parameter name."""
        names = {id(p): n for n, p in self.module.named_parameters()}
        for g in self.groups:
            full = torch.zeros(g.numel, dtype=torch.float32, device=self.device)
            full_now = self._gather_fp32(g, g.master)
            full.copy_(full_now)
            for p, o in zip(g.params, g.offsets):
                t = name_to_tensor.get(names[id(p)])
                if t is not None:
                    full[o:o + p.numel()] = t.reshape(-1).to(self.device, torch.float32)
            g.master.copy_(full[g.lo:g.hi])
            if g.sharded:
                g.param_shard.copy_(full[g.lo:g.hi].to(self.compute_dtype))
            else:
                g.flat_param.copy_(full.to(self.compute_dtype))
        if self.zero3:
            self._powner = [None, None]


import contextlib as _contextlib

_null_context = _contextlib.nullcontext

_HAS_FUSED_CPU_ADAMW = hasattr(torch, "_fused_adamw_")


class ShardedAdamW:
    """AdamW over a ``ParamStore`` (torch.optim.AdamW semantics, decoupled weight decay) with
    global-norm clipping folded in. ``state_dict`` follows torch's AdamW schema so checkpoints are
    interchangeable with the reference's (lset/train/checkpoint.py:9-53)."""

    def __init__(self, store: ParamStore, lr: float = 2e-5, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, grad_clip: float = 0.0):
        self.store = store
        self.defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.param_groups = [dict(self.defaults, params=list(store.trainable_parameters()),
                                  initial_lr=lr)]
        self.grad_clip = grad_clip
        self.step_count = 0
        dev = store.device
        # [squared global gradient norm, fault flag (sum of the ranks' status words)]
        self._sumsq = torch.zeros(2, dtype=torch.float32, device=dev)
        self._parts = torch.zeros(2, dtype=torch.float32, device=dev)
        # [clip coefficient, norm, skip flag]
        self._coef = torch.tensor([1.0, 0.0, 0.0], dtype=torch.float32, device=dev)
        self.state = {}  # torch.optim.Optimizer API expected by LR schedulers

    # -- torch.optim-like surface ------------------------------------------------------------
    def zero_grad(self, set_to_none: bool = True) -> None:
        self.store.zero_grad()

    @property
    def lr(self) -> float:
        return self.param_groups[0]["lr"]

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last ``step`` (device scalar)."""
        return self._coef[1]

    def _global_sumsq(self) -> None:
        """Squared global gradient norm into ``self._sumsq``: shards of tensor-parallel parameters
        are summed over the tensor-parallel group, replicated ones counted once, then everything is
        summed over the data-parallel shards."""
        st = self.store
        native = st.device.type == "cuda"
        parts = self._parts
        parts.zero_()
        if st.use_symm and not st.zero3:
            parts.copy_(st.sumsq)  # accumulated by the reduce kernels
        else:
            for g in st.groups:
                slot = 1 if getattr(g, "tp_sharded", False) else 0
                if native:
                    lib = nv.load()
                    scr = scratch("sumsq", lib.lb_sumsq_partial_rows(), st.device)
                    rc = lib.lb_sumsq_f32(nv.c_void_p(g.grad_shard.data_ptr()),
                                          nv.c_ll(g.grad_shard.numel()), nv.c_void_p(scr.data_ptr()),
                                          nv.c_void_p(parts.data_ptr() + 4 * slot), nv.c_int(1),
                                          nv.c_void_p(nv.stream_ptr()))
                    nv.check_rc(rc, "lb_sumsq_f32")
                    nv.count_launch(2)
                else:
                    gs = g.grad_shard.reshape(-1).float()
                    parts[slot] += torch.dot(gs, gs)       # one pass, no temporary
        tp_on = st.tp_group is not None and dist.get_world_size(st.tp_group) > 1
        if tp_on:
            dist.all_reduce(parts[1:2], op=dist.ReduceOp.SUM, group=st.tp_group)
        torch.sum(parts, dim=0, keepdim=True, out=self._sumsq[0:1])
        if native:
            # the status word of the bounded waits rides along: non-zero on any rank marks the
            # step as faulted on every rank (same reduction as the norm, no extra collective)
            self._sumsq[1:2].copy_(nv.status_word(st.device))
            if tp_on:
                dist.all_reduce(self._sumsq[1:2], op=dist.ReduceOp.SUM, group=st.tp_group)
        if st.world > 1:
            dist.all_reduce(self._sumsq, op=dist.ReduceOp.SUM, group=st.dp_group)

    @torch.no_grad()
    def step(self) -> None:
        st = self.store
        st.wait_reductions()
        self.step_count += 1
        pg = self.param_groups[0]
        lr, (b1, b2), eps, wd = pg["lr"], pg["betas"], pg["eps"], pg["weight_decay"]
        bc1 = 1.0 - b1 ** self.step_count
        bc2s = math.sqrt(1.0 - b2 ** self.step_count)
        self._global_sumsq()
        native = st.device.type == "cuda"
        if native:
            rc = nv.load().lb_clip_coef(nv.c_void_p(self._sumsq.data_ptr()), nv.c_float(self.grad_clip),
                                        nv.c_void_p(self._coef.data_ptr()),
                                        nv.c_void_p(self._sumsq.data_ptr() + 4),
                                        nv.c_void_p(nv.stream_ptr()))
            nv.check_rc(rc, "lb_clip_coef")
            nv.count_launch()
        else:
            norm = self._sumsq[0:1].sqrt()
            self._coef[1] = norm[0]
            self._coef[0] = torch.clamp(self.grad_clip / (norm[0] + 1e-6), max=1.0) \
                if self.grad_clip > 0 else 1.0
        for g in st.groups:
            pshard = g.param_shard if g.sharded else g.flat_param[g.lo:g.hi]
            if st.use_symm and not g.sharded:
                rc = nv.load().lb_adamw_push(
                    nv.c_void_p(g.master.data_ptr()), nv.c_void_p(g.grad_shard.data_ptr()),
                    nv.c_void_p(g.exp_avg.data_ptr()), nv.c_void_p(g.exp_avg_sq.data_ptr()),
                    g.symm_param.c_ptr_array(), nv.c_int(st.world), nv.c_int(st.rank), nv.c_ll(g.lo),
                    nv.c_ll(g.shard_numel), nv.c_float(lr), nv.c_float(b1), nv.c_float(b2),
                    nv.c_float(eps), nv.c_float(wd), nv.c_float(bc1), nv.c_float(bc2s),
                    nv.c_void_p(self._coef.data_ptr()), nv.c_void_p(nv.stream_ptr()))
                nv.check_rc(rc, "lb_adamw_push")
                nv.count_launch()
            elif native:
                rc = nv.load().lb_adamw_f32(
                    nv.c_void_p(g.master.data_ptr()), nv.c_void_p(g.grad_shard.data_ptr()),
                    nv.c_void_p(g.exp_avg.data_ptr()), nv.c_void_p(g.exp_avg_sq.data_ptr()),
                    nv.c_void_p(pshard.data_ptr() if g.compute_dtype == torch.bfloat16 else 0),
                    nv.c_ll(g.shard_numel), nv.c_float(lr), nv.c_float(b1), nv.c_float(b2),
                    nv.c_float(eps), nv.c_float(wd), nv.c_float(bc1), nv.c_float(bc2s),
                    nv.c_float(1.0), nv.c_void_p(self._coef.data_ptr()), nv.c_int(0),
                    nv.c_void_p(nv.stream_ptr()))
                nv.check_rc(rc, "lb_adamw_f32")
                nv.count_launch()
                if g.compute_dtype != torch.bfloat16:
                    pshard.copy_(g.master)
            elif _HAS_FUSED_CPU_ADAMW and g.master.dtype == torch.float32:
                # torch's single-pass CPU kernel (same update rule); the gradient shard is consumed
                # by this step, so the clip coefficient is applied to it in place
                if self.grad_clip > 0:
                    g.grad_shard.mul_(self._coef[0])
                torch._fused_adamw_([g.master], [g.grad_shard], [g.exp_avg], [g.exp_avg_sq], [],
                                    [torch.tensor(float(self.step_count))], lr=float(lr), beta1=b1,
                                    beta2=b2, weight_decay=wd, eps=eps, amsgrad=False,
                                    maximize=False)
                pshard.copy_(g.master)
            else:
                grad = g.grad_shard * self._coef[0]
                g.master.mul_(1.0 - lr * wd)
                g.exp_avg.mul_(b1).add_(grad, alpha=1.0 - b1)
                g.exp_avg_sq.mul_(b2).addcmul_(grad, grad, value=1.0 - b2)
                denom = g.exp_avg_sq.sqrt().div_(bc2s).add_(eps)
                g.master.addcdiv_(g.exp_avg, denom, value=-lr / bc1)
                pshard.copy_(g.master)
        st.gather_params()

    # -- checkpoint schema ---------------------------------------------------------------------
    def state_dict(self) -> dict:
        """torch AdamW layout: per-parameter ``step / exp_avg / exp_avg_sq`` (full tensors; a
        collective when world > 1) plus ``param_groups`` with integer parameter ids."""
        st = self.store
        canon = st.canonical_index()
        state = {}
        step_t = torch.tensor(float(self.step_count))
        for g in st.groups:
            m = st._gather_fp32(g, g.exp_avg)
            v = st._gather_fp32(g, g.exp_avg_sq)
            for p, o in zip(g.params, g.offsets):
                state[canon[id(p)]] = {"step": step_t.clone(),
                                       "exp_avg": m[o:o + p.numel()].view(p.shape).clone(),
                                       "exp_avg_sq": v[o:o + p.numel()].view(p.shape).clone()}
        state = dict(sorted(state.items()))
        pg = {k: v for k, v in self.param_groups[0].items() if k != "params"}
        pg.update(amsgrad=False, maximize=False, foreach=None, capturable=False,
                  differentiable=False, fused=True, params=list(range(len(state))))
        return {"state": state, "param_groups": [pg]}

    def load_state_dict(self, sd: dict) -> None:
        st = self.store
        canon = st.canonical_index()
        for g in st.groups:
            m = torch.zeros(g.numel, dtype=torch.float32, device=st.device)
            v = torch.zeros(g.numel, dtype=torch.float32, device=st.device)
            for p, o in zip(g.params, g.offsets):
                idx = canon[id(p)]
                ent = sd["state"].get(idx, sd["state"].get(str(idx)))
                if ent is not None:
                    m[o:o + p.numel()] = ent["exp_avg"].reshape(-1).to(st.device, torch.float32)
                    v[o:o + p.numel()] = ent["exp_avg_sq"].reshape(-1).to(st.device, torch.float32)
                    self.step_count = int(float(ent["step"]))
            g.exp_avg.copy_(m[g.lo:g.hi])
            g.exp_avg_sq.copy_(v[g.lo:g.hi])
        if sd.get("param_groups"):
            for k in ("lr", "betas", "eps", "weight_decay", "initial_lr"):
                if k in sd["param_groups"][0]:
                    val = sd["param_groups"][0][k]
                    self.param_groups[0][k] = tuple(val) if k == "betas" else val
