"""Arrangement of a layer's parts: the pre-norm residual block.

``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/engine/batched_engine.ts:800-1314).
Each sublayer's output is left pending on the residual stream and folded in by
the next norm, this layer's or the following one's.
"""
from __future__ import annotations

from typing import List

from ..config.specs import LayerSpec, NameLayout
from .base import (BuildEnv, EntryView, Part, ResidualStream, StepContext, build_ffn,
                   build_mixer, build_norm, register_block)


class PreNormBlock(Part):
    def __init__(self, spec: LayerSpec, hidden_size: int, names: NameLayout, index: int,
                 env: BuildEnv):
        p = names.layer_prefix.format(i=index)
        self.index = index
        self.input_norm = build_norm(spec.norm, hidden_size, f"{p}{names.input_norm}.weight", env)
        self.mixer = build_mixer(spec.mixer, hidden_size, f"{p}{names.mixer}.", env)
        self.post_norm = build_norm(spec.norm, hidden_size,
                                    f"{p}{names.post_mixer_norm}.weight", env)
        self.ffn = build_ffn(spec.ffn, hidden_size, f"{p}{names.ffn}.", env)

    def parts(self) -> List[Part]:
        return [self.input_norm, self.mixer, self.post_norm, self.ffn]

    def param_specs(self):
        return [s for part in self.parts() for s in part.param_specs()]

    def load(self, get) -> None:
        for part in self.parts():
            part.load(get)

    def forward(self, stream: ResidualStream, ctx: StepContext, view: EntryView) -> None:
        stream.add(self.mixer.forward(self.input_norm.forward(stream), ctx, view))
        stream.add(self.ffn.forward(self.post_norm.forward(stream), ctx))


register_block("prenorm", PreNormBlock)
