"""The parts a model is put together from, their interfaces and registries."""
from .base import (Block, Branch, BuildEnv, FeedForward, KvNeed, Mixer, Norm, Part, PositionEncoding,
                   StateNeed, TensorDecl, part_class, register_part, unregister_part)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = ["Block", "Branch", "BuildEnv", "FeedForward", "KvNeed", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateNeed", "TensorDecl", "part_class", "register_part", "unregister_part",
           "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry"]
