"""The dense matrix product ``y = x W^T`` with weights as stored (``[out, in]`` row-major).

float32 engine: the engine's own FP32-FMA kernel (no reduced-precision matrix mode).
bfloat16 engine: cuBLAS through ``torch.mm`` with float accumulation, the same
library call the reference makes for every dense product
(cuda/kernels/gemm.cu:244-267: ``cublasGemmEx``, bf16 in, ``CUBLAS_COMPUTE_32F``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


def linear(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T -> [M, N]``; ``out_dtype`` float32 keeps a bfloat16
    product's accumulator precision (used for the logits)."""
    M, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32:
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        ops.sgemm_nt(x, w, out)
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError(f"linear: unsupported dtypes {x.dtype} x {w.dtype}")
    prof = ops._profiler
    if prof is not None:
        prof.begin("cublas_gemm_bf16")
    ops.count_library_launch()
    if out_dtype == torch.float32:
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    elif out is None:
        out = torch.mm(x, w.t())
    else:
        torch.mm(x, w.t(), out=out)
    if prof is not None:
        prof.end("cublas_gemm_bf16")
    return out
