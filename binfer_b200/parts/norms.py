"""RMSNorm over the residual stream, fused with the stream's pending add.

``y = x * rsqrt(mean(x^2) + eps) * w`` with the weight multiplying directly
(cuda/kernels/bf16_kernels.cu:40-84).  The reference runs the residual add and
the norm as two kernels (src/engine/batched_engine.ts:1164-1178); here the add
rides on the norm.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..config.specs import NormSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, Norm, ResidualStream, register_norm


class RMSNorm(Norm):
    def __init__(self, spec: NormSpec, size: int, name: str, env: BuildEnv):
        self.eps = float(spec.eps)
        self.size = size
        self.name = name
        self.env = env
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name, (self.size,), init="norm", role="vector")]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        self.weight = get(self.param_specs()[0])

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                n_rows: int = 0) -> torch.Tensor:
        """Normed activations of every row, or of ``rows`` only (the stream is then
        left as it is: nothing reads it afterwards).  May return ``ScaledRows`` when the
        stream holds this norm's output already (``ResidualStream.add_linear``)."""
        if rows is None and stream.ready_for is self:
            out, stream.ready, stream.ready_for = stream.ready, None, None
            return out           # ScaledRows: the product before already prepared this norm
        stream.ready = stream.ready_for = None
        n = n_rows if rows is not None else stream.x.shape[0]
        out = torch.empty((n, self.size), dtype=self.env.dtype, device=self.env.device)
        ops.add_rmsnorm(stream.x, stream.pending, self.weight, out, self.eps, rows=rows,
                        write_back=rows is None)
        if rows is None:
            stream.pending = None
        return out


    def fused_scale(self):
        """(weight, eps): what a product needs to prepare this norm in its epilogue."""
        return self.weight, self.eps


register_norm("rmsnorm", RMSNorm)
