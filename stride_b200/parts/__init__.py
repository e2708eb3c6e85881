from .base import (Block, BranchScale, BuildEnv, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Rewrite, part_class,
                   register_part)
from .context import ResidualStream, StepContext, Workspace
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorPlan
from . import (attention, block, branch, ends, experts, hgrn2, lightning, masked_attention, mlp, norm, parallel, reentry, rglru,  # register the
               rope, sigmoid_attention)                                                                                       # built-in kinds
from .model import DecoderModel

__all__ = ["Block", "BranchScale", "BuildEnv", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Rewrite", "part_class",
           "register_part", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "TensorPlan", "DecoderModel", "ResidualStream", "StepContext", "Workspace"]
