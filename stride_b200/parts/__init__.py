from .base import (Block, BranchScale, BuildEnv, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Rewrite, part_class,
                   register_part)
from .context import ResidualStream, StepContext, Workspace
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorPlan
from . import (attention, block, branch, ends, experts, gated_attention, gated_delta, hgrn2, lightning, masked_attention, mlp, norm,  # register the
               parallel, reentry, retention, rglru, rope, sigmoid_attention, token_side)                                              # built-in kinds
from .model import DecoderModel

__all__ = ["Block", "BranchScale", "BuildEnv", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Rewrite", "part_class",
           "register_part", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "TensorPlan", "DecoderModel", "ResidualStream", "StepContext", "Workspace"]
