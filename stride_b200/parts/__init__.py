from .base import (Block, BuildEnv, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Rewrite, part_class,
                   register_part)
from .context import ResidualStream, StepContext, Workspace
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorPlan
from . import attention, block, ends, lightning, mlp, norm, reentry, rope  # register the built-in kinds
from .model import DecoderModel

__all__ = ["Block", "BuildEnv", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Rewrite", "part_class",
           "register_part", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "TensorPlan", "DecoderModel", "ResidualStream", "StepContext", "Workspace"]
