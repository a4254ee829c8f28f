"""Dense gated feed-forward (SwiGLU): ``down( silu(gate(x)) * up(x) )``.

``silu(g) = g / (1 + exp(-g))`` (cuda/kernels/bf16_kernels.cu:461-477).  The
reference runs gate and up as two products (src/engine/batched_engine.ts:1243-1244);
here they are one product against the stacked weight ``[2 I, H]``, and the
activation kernel reads both halves of each output row.
"""
from __future__ import annotations

import os
from typing import Callable, List

import torch

from ..config.specs import GatedMLPSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import (BuildEnv, DeferredLinear, FeedForward, ScaledRows, StepContext, register_ffn,
                   split_scaled)
from .linear import linear, pair_token_limit, swiglu_token_limit

# BINFER_B200_FUSE_SWIGLU=0: the stacked gate/up projection and the activation as two kernels
FUSE_SWIGLU = os.environ.get("BINFER_B200_FUSE_SWIGLU", "1") != "0"
# ... and only where its tiles (at least 16 outputs each) give work to this share of the SMs
FUSE_SWIGLU_FILL = 0.5


class GatedMLP(FeedForward):
    def __init__(self, spec: GatedMLPSpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported (supported: 'silu')")
        if spec.bias:
            raise ValueError("feed-forward biases are not supported")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.inter = spec.intermediate_size
        self.w_gate_up = self.w_down = None
        self._swiglu_plan = None

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
        h = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        if not self._project_fused(x, h, row_scale):
            gu = linear(x, self.w_gate_up)
            ops.silu_mul(gu, h, row_scale=row_scale)
        return DeferredLinear(h, self.w_down)

    def _project_fused(self, x, h, row_scale) -> bool:
        """Few token rows in bfloat16: the stacked projection with the activation in its
        epilogue, one CTA a tile of gate rows and the up rows of the same outputs.  False,
        having done nothing, where that kernel does not run."""
        if not FUSE_SWIGLU or x.dtype != torch.bfloat16 or self.inter % 8:
            return False
        pair_from = pair_token_limit()
        if pair_from and x.shape[0] >= pair_from and row_scale is None:
            # many token rows: the product on pairs of SMs, the activation in its epilogue
            return ops.gemm_bf16_pair(x, self.w_gate_up, h, ops.error_word(x.device), gated=True)
        if x.shape[0] > swiglu_token_limit():
            return False
        if self._swiglu_plan is None:
            self._swiglu_plan = ops.gemm_swiglu_plan(self.inter, x.shape[1], x.device) or False
        plan = self._swiglu_plan
        if not plan or plan[1] < FUSE_SWIGLU_FILL * ops.num_sms(x.device):
            return False
        return ops.gemm_bf16_swiglu(x, self.w_gate_up, h, ops.error_word(x.device), plan[0],
                                    row_scale=row_scale)


register_ffn("gated_mlp", GatedMLP)
