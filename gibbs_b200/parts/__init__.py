from .base import (Residual, Block, FeedForward, Mixer, Norm, PagedKV, Part, PositionEncoding, Rotary, Runtime, SlotState,
                   TensorDecl, MATRIX, VECTOR, INT_TABLE, part_class, register_part)
from . import norm, position, attention, short_conv, ffn, block, embedding  # noqa: F401  (register the built-in kinds)
from .linear import Linear
from .model import CausalLM, build_model

__all__ = ["Residual", "Block", "FeedForward", "Mixer", "Norm", "PagedKV", "Part", "PositionEncoding", "Rotary", "Runtime",
           "SlotState", "TensorDecl", "MATRIX", "VECTOR", "INT_TABLE", "part_class", "register_part", "Linear",
           "CausalLM", "build_model"]
