"""nabla_b200: B200 (sm_100a) implementation of nabla-train's optimizer-step path.

The product is ``libnabla_optim_b200.so`` (C ABI in ``include/nabla_optim_b200.h``);
this package is the Python host mirror of the reference's Rust interface on top of it.
"""
from .optim import (Adam, AdamW, GradClipper, GradScaler, GroupOptimizer, LrSchedule, MixedAdamW,
                    Optimizer, ParamExclusionPreset, ParamGroupConfig, ParamMatch, ParamSelector, Sgd,
                    StepOutcome, adamw_step, assign_groups, clip_grad_norm, lr_at_step)
from . import checkpoint
from .trainer import GradAccumulator, GradNanPolicy, NonFiniteGradient, TrainerTail
from .zero1 import Zero1AdamW, exchange_unique_id, geometry, shard_pieces

__all__ = [
    "Adam", "AdamW", "GradAccumulator", "GradClipper", "GradNanPolicy", "NonFiniteGradient", "TrainerTail", "GradScaler", "GroupOptimizer", "LrSchedule", "MixedAdamW", "Optimizer",
    "ParamExclusionPreset", "ParamGroupConfig", "ParamMatch", "ParamSelector", "Sgd", "StepOutcome",
    "Zero1AdamW", "adamw_step", "assign_groups", "clip_grad_norm", "exchange_unique_id", "geometry", "lr_at_step",
    "shard_pieces",
]
