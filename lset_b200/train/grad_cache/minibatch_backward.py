"""Runtime policies for the GradCache replay: how to run several backward passes per optimizer
step without reducing gradients every time, for each kind of data-parallel runtime.

``MinibatchBackward.for_model(obj)`` picks a policy by duck typing, like the reference
(lset/train/grad_cache/minibatch_backward.py:69-227):
  * ``ParamStore`` of this framework   -> gradient reduction off while replaying, on for the last
                                           minibatch of an accumulation boundary
  * ``DistributedDataParallel``        -> ``no_sync()`` + one flat all-reduce per dtype at the end
  * FSDP2-style module                 -> ``set_requires_gradient_sync`` toggling
  * DeepSpeed-style engine             -> ``set_gradient_accumulation_boundary`` + ``engine.backward``
  * anything else                      -> plain ``backward``
``align_minibatches`` pads every rank's plan to the longest one (all-reduce MAX) so all ranks run
the same number of forwards and therefore the same sequence of collectives.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import Iterable, List, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .planner import Range


def _dist_on(group=None) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


class MinibatchBackward:
    group = None

    @classmethod
    def for_model(cls, obj, *, is_ga_boundary: bool = True, store=None) -> "MinibatchBackward":
        from ...dist.sharded import ParamStore

        if store is not None or isinstance(obj, ParamStore):
            return ShardedStoreMinibatchBackward(store if store is not None else obj, is_ga_boundary)
        if all(hasattr(obj, a) for a in ("set_gradient_accumulation_boundary", "backward", "module")):
            return DeepSpeedMinibatchBackward(obj, is_ga_boundary)
        if isinstance(obj, nn.parallel.DistributedDataParallel):
            return DDPMinibatchBackward(obj, is_ga_boundary)
        if hasattr(obj, "set_requires_gradient_sync") and hasattr(obj, "set_reshard_after_backward"):
            return FSDP2MinibatchBackward(obj, is_ga_boundary)
        return BasicMinibatchBackward()

    def context(self):
        return nullcontext()

    def backward(self, surrogate: torch.Tensor, is_last: bool) -> None:
        raise NotImplementedError

    def finalize(self, params: Iterable[nn.Parameter]) -> None:
        return None

    def align_minibatches(self, plans: List[List[Range]]) -> Tuple[List[List[Range]], List[int]]:
        """Returns (padded plans, real lengths). Padding repeats the last real range; the caller
        runs those with a zero gradient."""
        real = [len(p) for p in plans]
        if not _dist_on(self.group):
            return plans, real
        dev = "cuda" if dist.get_backend(self.group) == "nccl" else "cpu"
        t = torch.tensor(real, dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        out = []
        for p, want in zip(plans, t.tolist()):
            out.append(list(p) + [p[-1]] * (want - len(p)) if p else p)
        return out, real


class BasicMinibatchBackward(MinibatchBackward):
    def backward(self, surrogate, is_last):
        surrogate.backward()


class ShardedStoreMinibatchBackward(MinibatchBackward):
    def __init__(self, store, is_ga_boundary: bool = True):
        self.store, self.is_ga_boundary = store, is_ga_boundary
        self.group = store.dp_group

    def backward(self, surrogate, is_last):
        self.store.set_requires_gradient_sync(bool(is_last and self.is_ga_boundary))
        surrogate.backward()

    def finalize(self, params):
        self.store.set_requires_gradient_sync(self.is_ga_boundary)


class FSDP2MinibatchBackward(MinibatchBackward):
    def __init__(self, module, is_ga_boundary: bool = True):
        self.module, self.is_ga_boundary = module, is_ga_boundary

    def backward(self, surrogate, is_last):
        self.module.set_requires_gradient_sync(bool(is_last and self.is_ga_boundary))
        surrogate.backward()

    def finalize(self, params):
        self.module.set_requires_gradient_sync(True)


class DDPMinibatchBackward(MinibatchBackward):
    def __init__(self, ddp, is_ga_boundary: bool = True):
        self.ddp, self.is_ga_boundary = ddp, is_ga_boundary

    def context(self):
        return self.ddp.no_sync()

    def backward(self, surrogate, is_last):
        surrogate.backward()

    def finalize(self, params):
        if not (self.is_ga_boundary and _dist_on()):
            return
        by_dtype = {}
        for p in params:
            if p.grad is not None:
                by_dtype.setdefault(p.grad.dtype, []).append(p)
        world = dist.get_world_size()
        for ps in by_dtype.values():
            flat = torch.cat([p.grad.reshape(-1) for p in ps])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM)
            flat.div_(world)
            off = 0
            for p in ps:
                n = p.grad.numel()
                p.grad.copy_(flat[off:off + n].view_as(p.grad))
                off += n


class DeepSpeedMinibatchBackward(MinibatchBackward):
    def __init__(self, engine, is_ga_boundary: bool = True):
        self.engine, self.is_ga_boundary = engine, is_ga_boundary

    def backward(self, surrogate, is_last):
        self.engine.set_gradient_accumulation_boundary(bool(is_last and self.is_ga_boundary))
        self.engine.backward(surrogate)
