"""Parts a layer is put together from, their registries, and the decoder that runs them."""
from .base import (BuildEnv, EntryView, FeedForward, Mixer, Norm, Part, PositionEncoding,
                   ResidualStream, StepContext, build_block, build_ffn, build_mixer,
                   build_norm, build_position, register_block, register_ffn, register_mixer,
                   register_norm, register_position)
from .linear import linear
from .model import DecoderModel, build_model, param_specs_for

__all__ = [
    "BuildEnv", "EntryView", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
    "ResidualStream", "StepContext", "build_block", "build_ffn", "build_mixer", "build_norm",
    "build_position", "register_block", "register_ffn", "register_mixer", "register_norm",
    "register_position", "linear", "DecoderModel", "build_model", "param_specs_for",
]
