"""The dense matrix product ``y = x W^T`` with weights as stored (``[out, in]`` row-major).

float32 engine: the engine's own FP32-FMA kernel (no reduced-precision matrix mode).
bfloat16 engine: the engine's tcgen05/TMEM/TMA kernel (``csrc/gemm_tcgen05.cu``) or
cuBLAS through ``torch.mm`` with float accumulation, the library call the reference
makes for every dense product (cuda/kernels/gemm.cu:244-267: ``cublasGemmEx``, bf16
in, ``CUBLAS_COMPUTE_32F``).  Which one: ``BINFER_B200_GEMM=own`` takes the engine's
kernel for every shape it accepts, ``library`` never, and ``auto`` (the default)
where it was measured to be at least as fast as the library on a B200: at most 128
tokens against a very wide weight (the output head while decoding), and at most 32
tokens against a weight of at most 8192 output features, where the split-K cluster
kernel (``csrc/gemm_tcgen05_cluster.cu``) runs (the qkv, output and down projections).
Alone, the cluster kernel ties with the library on the qkv projection; inside a decode
step it wins, because it is launched as a programmatic dependent of the kernel before
it and has its first weight tiles under way when that kernel ends.
"""
from __future__ import annotations

from typing import Optional

import os

import torch

from ..csrc import ops

_POLICY = os.environ.get("BINFER_B200_GEMM", "auto")


def set_gemm_policy(policy: str) -> None:
    """``own``, ``library`` or ``auto`` (see the module text)."""
    global _POLICY
    if policy not in ("own", "library", "auto"):
        raise ValueError(f"unknown GEMM policy {policy!r}")
    _POLICY = policy


def _use_own(M: int, N: int, K: int) -> bool:
    if _POLICY == "own":
        return True
    if _POLICY == "library":
        return False
    return M <= 128 and N >= 65536


# Fewest token rows from which the gated feed-forward product goes to the kernel on pairs of
# SMs (``csrc/gemm_tcgen05_pair.cu``, the activation in its epilogue).  Measured against the
# library's product followed by the activation kernel, 12288 outputs from 4096 inputs:
# 54 against 41 us at 128 tokens, 56 / 53 at 256, 82 / 82 at 512, 152 to 165 / 155 at 1024
# (a tie within the runs' scatter), 276 / 303 at 2048, 515 / 590 at 4096; 6144 outputs from 2048
# inputs: 83 / 83 at 2048, 138 / 165 at 4096; 25600 from 5120: 355 / 381 at 1024, 678 / 772 at
# 2048.  0: never.
_PAIR_MIN_TOKENS = int(os.environ.get("BINFER_B200_PAIR_MIN_TOKENS", "1024"))
# The plain products stay with the library under "auto": the pair kernel takes 74 / 50 / 148 us
# where the library takes 71 / 46 / 136 (2048 tokens; q/k/v, output and down projection).
_PAIR_PLAIN = os.environ.get("BINFER_B200_PAIR_PLAIN", "0") != "0"


def pair_token_limit() -> int:
    """Fewest token rows for which the gated product goes to the kernel on pairs of SMs
    (0: never)."""
    if _POLICY == "library":
        return 0
    return _PAIR_MIN_TOKENS if _POLICY == "auto" else 256


def _use_pair(M: int, N: int, K: int) -> bool:
    lim = pair_token_limit()
    return (_PAIR_PLAIN or _POLICY == "own") and lim > 0 and M >= lim and 1024 <= N < 65536


def _use_cluster(M: int, N: int, K: int) -> bool:
    # (at 24 tokens the library takes 6.14 against the kernel's 5.98 ms, at 32: 6.96 against 6.97)
    if _POLICY == "library" or M > cluster_token_limit():
        return False
    # wider weights (the gate/up projection, on "clusters" of one CTA) measured 2 us slower
    # per call than the library inside a decode step
    return N <= (_CLUSTER_MAX_FEATURES if _POLICY == "auto" else 32768) and (
        K >= 2048 or _POLICY == "own")


# widest weight (output features) that goes to the cluster kernel under "auto"
_CLUSTER_MAX_FEATURES = int(os.environ.get("BINFER_B200_CLUSTER_MAX_FEATURES", "8192"))


# most token rows that go to the cluster kernel under "auto".  The kernel takes 64 (64-row
# products with all four lane quarters of tensor memory in use), but from 33 rows on the
# library is faster inside a step, all 36 layers, 16-token pages: 7.31 against 7.45 ms at 33
# tokens, 8.97 against 9.31 at 48, 10.87 against 11.39 at 64 (library against own; clusters
# of 2 or 1 instead of 4: 11.71 and 13.85).  With 64 token rows a ring slot is 24 KB and the
# partial sums' landing area 32 KB, which leaves 6 slots: 96 KB of weights in flight per SM,
# against 160 KB at 16 rows.
_CLUSTER_MAX_TOKENS = int(os.environ.get("BINFER_B200_CLUSTER_MAX_TOKENS", "32"))


# ... and for the gate/up projection with the activation in its epilogue (the same kernel, on
# "clusters" of one CTA).  Inside a step against the library's product followed by the
# activation kernel: a tie from 33 to 56 rows (7.06 / 7.07 ms at 33, 8.72 / 8.69 at 48,
# 9.62 / 9.62 at 56), 10.45 against 10.56 ms at 64.  The other three products at 64 rows each
# cost 0.2 ms a step against the library (10.75 to 10.80 ms).
_SWIGLU_MAX_TOKENS = int(os.environ.get("BINFER_B200_SWIGLU_MAX_TOKENS", "64"))


def swiglu_token_limit() -> int:
    """Most token rows for which the gate/up projection runs on the cluster kernel's gated form."""
    if _POLICY == "library":
        return 0
    return min(_SWIGLU_MAX_TOKENS, ops.CLUSTER_MAX_TOKENS) if _POLICY == "auto" \
        else ops.CLUSTER_MAX_TOKENS


def cluster_token_limit() -> int:
    """Most token rows for which the policy sends products to the split-K cluster kernel."""
    if _POLICY == "library":
        return 0
    return min(_CLUSTER_MAX_TOKENS, ops.CLUSTER_MAX_TOKENS) if _POLICY == "auto" \
        else ops.CLUSTER_MAX_TOKENS


_plans = {}


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
    K = x.shape[1]
    if _use_cluster(M, N, K):
        plan = _plans.get((N, K))
        if plan is None:
            plan = _plans[(N, K)] = ops.gemm_cluster_plan(N, K, x.device) or False
        if plan:
            if out is None:
                out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
            if ops.gemm_bf16_cluster(x, w, out, ops.error_word(x.device), *plan):
                return out
    if _use_pair(M, N, K):
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
        if ops.gemm_bf16_pair(x, w, out, ops.error_word(x.device)):
            return out
    if _use_own(M, N, K):
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
        if ops.gemm_bf16(x, w, out, ops.error_word(x.device)):
            return out
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


FUSE_NORM = os.environ.get("BINFER_B200_FUSE_NORM", "1") != "0"


def linear_add_norm(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor,
                    norm_w: torch.Tensor, eps: float):
    """``resid += x @ w^T`` with the next RMSNorm prepared in the same kernel: returns
    ``(bfloat16(resid * norm_w), ops.RowScale)``, the norm's output short of the factor
    ``rsqrt(mean(resid^2) + eps)`` per row, or None, having done nothing, where the cluster
    kernel does not run (float32, more than 32 tokens, shapes without a plan)."""
    M, (N, K) = x.shape[0], w.shape
    if (not FUSE_NORM or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
            or not _use_cluster(M, N, K)):
        return None
    plan = _plans.get((N, K))
    if plan is None:
        plan = _plans[(N, K)] = ops.gemm_cluster_plan(N, K, x.device) or False
    if not plan:
        return None
    return ops.gemm_bf16_cluster_add_norm(x, w, resid, norm_w, eps, ops.error_word(x.device),
                                          *plan)

