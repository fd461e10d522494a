"""The parts layers are assembled from.  Importing this package registers the built-in
kinds: norm "rmsnorm", position "rope", mixer "attention", ffn "swiglu", block "prenorm",
head "linear"."""
from .base import (Block, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Runtime, StepContext, StepInput,
                   Workspace, part_class, register_part, unregister_part)
from .linear import Linear
from . import norm, rope, attention, swiglu, block, head  # noqa: F401  (registration)

__all__ = ["Block", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
           "StepContext", "StepInput", "Workspace", "part_class", "register_part", "unregister_part", "Linear"]
