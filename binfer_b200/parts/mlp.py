"""Dense gated feed-forward (SwiGLU): ``down( silu(gate(x)) * up(x) )``.

``silu(g) = g / (1 + exp(-g))`` (cuda/kernels/bf16_kernels.cu:461-477).  The
reference runs gate and up as two products (src/engine/batched_engine.ts:1243-1244);
here they are one product against the stacked weight ``[2 I, H]``, and the
activation kernel reads both halves of each output row.
"""
from __future__ import annotations

from typing import Callable, List

import torch

from ..config.specs import GatedMLPSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import (BuildEnv, DeferredLinear, FeedForward, ScaledRows, StepContext, register_ffn,
                   split_scaled)
from .linear import linear


class GatedMLP(FeedForward):
    def __init__(self, spec: GatedMLPSpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported (supported: 'silu')")
        if spec.bias:
            raise ValueError("feed-forward biases are not supported")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.inter = spec.intermediate_size
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> List[ParamSpec]:
        p = self.prefix
        return [ParamSpec(p + "gate_proj.weight", (self.inter, self.hidden)),
                ParamSpec(p + "up_proj.weight", (self.inter, self.hidden)),
                ParamSpec(p + "down_proj.weight", (self.hidden, self.inter))]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g, u, d = self.param_specs()
        self.w_gate_up = torch.cat([get(g), get(u)], dim=0).contiguous()
        self.w_down = get(d)

    accepts_scaled_rows = True

    def forward(self, x, ctx: StepContext) -> torch.Tensor:
        return self.forward_deferred(x, ctx).compute()

    def forward_deferred(self, x, ctx: StepContext) -> DeferredLinear:
        """Everything but the down projection (see ``GQAAttention.forward_deferred``)."""
        if isinstance(x, ScaledRows) and (self.inter % 8 or self.inter < 256):
            x = x.dense()                  # the activation kernel takes the factor at other sizes only
        x, row_scale = split_scaled(x)
        gu = linear(x, self.w_gate_up)
        h = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.silu_mul(gu, h, row_scale=row_scale)
        return DeferredLinear(h, self.w_down)


register_ffn("gated_mlp", GatedMLP)
