from .minibatch_backward import MinibatchBackward
from .planner import plan_minibatches, slice_feature
from .rand_context import RandContext
from .wrapper import GradCacheWrapper

__all__ = ["GradCacheWrapper", "MinibatchBackward", "RandContext", "plan_minibatches",
           "slice_feature"]
