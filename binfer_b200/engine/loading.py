"""From a model folder (or a configuration and a seed) to a model and its runner.

Start-up in the reference: ``MmapModelLoader.load`` -> ``parseLlamaConfig`` ->
one ``cudaMalloc`` + copy per tensor (src/loader/mmap_loader.ts:47-83,175-225),
then the engine's constructor sizes the page pool from a memory figure
(src/kv/paged.ts:55-62).  Here the architecture is chosen by config.json through
the registry, and the pool is sized in pages or tokens by the caller.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from ..cache.manager import CacheManager
from ..config.registry import load_config
from ..parts.base import BuildEnv
from ..parts.model import DecoderModel, build_model, param_specs_for
from ..weights.loader import TensorSource
from ..weights.random_init import random_tensor
from .runner import ModelRunner

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, got {name}")
        return name
    if name not in _DTYPES:
        raise ValueError(f"unknown dtype {name!r} (bfloat16 or float32)")
    return _DTYPES[name]


def make_env(dtype: Union[str, torch.dtype], device: Union[str, torch.device] = "cuda:0") -> BuildEnv:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("the engine runs on a CUDA device only (there is no CPU path)")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; the engine has no CPU path")
    torch.cuda.set_device(device)
    return BuildEnv(parse_dtype(dtype), device)


def model_from_dir(model_dir: str, env: BuildEnv, allow_unexpected: bool = False) -> DecoderModel:
    config = load_config(model_dir)
    source = TensorSource.from_dir(model_dir)
    try:
        return build_model(config.to_spec(), env, source, allow_unexpected=allow_unexpected)
    finally:
        source.close()


def model_from_seed(config, env: BuildEnv, seed: int = 0, std: float = 0.02,
                    norm_std: float = 0.0) -> DecoderModel:
    """Random weights generated on the device, tensor by tensor (nothing is written)."""
    spec = config.to_spec()
    by_name = {s.name: s for s in param_specs_for(spec)}

    def get(name: str) -> torch.Tensor:
        s = by_name[name]
        dtype = torch.float32 if s.role == "vector" else env.dtype
        return random_tensor(s, seed, std, norm_std, dtype=dtype, device=env.device)

    source = TensorSource(get, {n: s.shape for n, s in by_name.items()}, where="(random)")
    return build_model(spec, env, source)


def make_runner(model: DecoderModel, env: BuildEnv, page_size: int = 16,
                num_pages: Optional[int] = None, max_tokens: Optional[int] = None,
                max_requests: int = 64) -> ModelRunner:
    """A runner whose page pool holds ``num_pages`` pages per cache group, or enough
    pages for ``max_tokens`` cached tokens."""
    if num_pages is None:
        if max_tokens is None:
            raise ValueError("give num_pages or max_tokens")
        num_pages = -(-int(max_tokens) // page_size)
    cache = CacheManager(model.kv_needs(), model.state_needs(), page_size=page_size,
                         num_pages=num_pages, max_requests=max_requests)
    return ModelRunner(model, cache, env)
