"""Rotary position encoding (rotate-half layout) as a part of the attention mixer.

``f_i = theta^(-2i/rot) / factor`` for ``i < rot/2``; a token at absolute
position ``p`` rotates the pair ``(i, i + rot/2)`` of each q and k head by the
angle ``p * f_i`` (src/engine/tp_context.ts:181-221;
cuda/kernels/bf16_kernels.cu:133-185).  The reference builds a cos/sin table for
4096 positions on the host and truncates it to bfloat16
(src/tensor/tensor.ts:136-145); here only the ``rot/2`` frequencies are kept, in
float32, and the kernel forms the angle and its sine and cosine in float32, so
no position limit and no table precision enter.
"""
from __future__ import annotations

import torch

from ..config.specs import RopeSpec
from .base import BuildEnv, PositionEncoding, register_position


class RotaryEncoding(PositionEncoding):
    """Holds ``inv_freq`` (float32 ``[rot/2]``) for the qkv post-processing kernel."""

    def __init__(self, spec: RopeSpec, head_dim: int, env: BuildEnv):
        rot = spec.rotary_dim or head_dim
        if rot % 2 or rot > head_dim:
            raise ValueError(f"rotary_dim {rot} must be even and at most head_dim {head_dim}")
        self.rotary_dim = rot
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = (float(spec.theta) ** (-2.0 * i / rot)) / float(spec.factor)
        self.inv_freq = inv.to(torch.float32).to(env.device)


register_position("rope", RotaryEncoding)
