"""Arrangement of a layer's parts: the pre-norm residual block.

``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/engine/batched_engine.ts:800-1314).
Each sublayer's output is left pending on the residual stream and folded in by
the next norm, this layer's or the following one's.
"""
from __future__ import annotations

from typing import List

from ..config.specs import LayerSpec, NameLayout
from .base import (BuildEnv, EntryView, Part, ResidualStream, ScaledRows, StepContext, build_ffn,
                   build_mixer, build_norm, register_block)


class PreNormBlock(Part):
    takes_successor = True      # forward(stream, ctx, view, successor): see DecoderModel.forward

    def __init__(self, spec: LayerSpec, hidden_size: int, names: NameLayout, index: int,
                 env: BuildEnv):
        p = names.layer_prefix.format(i=index)
        self.index = index
        self.input_norm = build_norm(spec.norm, hidden_size, f"{p}{names.norm('input')}.weight", env)
        self.mixer = build_mixer(spec.mixer, hidden_size, f"{p}{names.mixer}.", env)
        self.post_norm = build_norm(spec.norm, hidden_size,
                                    f"{p}{names.norm('post_mixer')}.weight", env)
        self.ffn = build_ffn(spec.ffn, hidden_size, f"{p}{names.ffn}.", env)

    def parts(self) -> List[Part]:
        return [self.input_norm, self.mixer, self.post_norm, self.ffn]

    def param_specs(self):
        return [s for part in self.parts() for s in part.param_specs()]

    def load(self, get) -> None:
        for part in self.parts():
            part.load(get)

    def forward(self, stream: ResidualStream, ctx: StepContext, view: EntryView,
                successor: "PreNormBlock" = None) -> None:
        """``successor``: the block that runs next on this stream, if any; its input norm
        can then be prepared by this block's last product."""
        h = self._for(self.mixer, self.input_norm.forward(stream))
        deferred = getattr(self.mixer, "forward_deferred", None)
        if deferred is not None:
            stream.add_linear(deferred(h, ctx, view), self.post_norm, self.ffn)
        else:
            stream.add(self.mixer.forward(h, ctx, view))
        h = self._for(self.ffn, self.post_norm.forward(stream))
        deferred = getattr(self.ffn, "forward_deferred", None)
        if deferred is not None:
            nxt = successor if isinstance(successor, PreNormBlock) else None
            stream.add_linear(deferred(h, ctx), nxt.input_norm if nxt else None,
                              nxt.mixer if nxt else None)
        else:
            stream.add(self.ffn.forward(h, ctx))

    @staticmethod
    def _for(part, h):
        """``h`` as ``part`` can take it."""
        if isinstance(h, ScaledRows) and not getattr(part, "accepts_scaled_rows", False):
            return h.dense()
        return h


register_block("prenorm", PreNormBlock)
