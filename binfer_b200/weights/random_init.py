"""Random-weights mode: tensors, or a whole model folder, from a configuration and a seed.

The reference has no such mode (it always loads a checkpoint,
src/loader/mmap_loader.ts:47-83).  Each tensor's values depend only on
(seed, tensor name), not on the order of generation, so a model built in
memory and one written to a folder and read back hold the same numbers.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Iterable, Optional

import torch

from .loader import ParamSpec
from .safetensors_io import save_file


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1_000_003 + zlib.crc32(name.encode("utf-8"))) & 0x7FFF_FFFF_FFFF


def random_tensor(spec: ParamSpec, seed: int, std: float, norm_std: float,
                  dtype: torch.dtype = torch.float32,
                  device: torch.device | str = "cpu") -> torch.Tensor:
    """``matrix``: N(0, std).  ``norm``: 1 + N(0, norm_std).  ``zeros``: 0."""
    device = torch.device(device)
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    x = torch.empty(spec.shape, dtype=torch.float32, device=device)
    if device.type == "cuda" and x.numel() > (1 << 28):
        # fill big tables in slices so the 32-bit staging stays small
        flat = x.view(-1)
        step = 1 << 27
        for a in range(0, flat.numel(), step):
            flat[a:a + step].normal_(0.0, 1.0, generator=g)
    else:
        x.normal_(0.0, 1.0, generator=g)
    if spec.init == "norm":
        x.mul_(norm_std).add_(1.0)
    else:
        x.mul_(std)
    return x.to(dtype)


def random_tensors(specs: Iterable[ParamSpec], seed: int, std: float = 0.02,
                   norm_std: float = 0.01, dtype: torch.dtype = torch.float32,
                   device: torch.device | str = "cpu") -> Dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, std, norm_std, dtype, device) for s in specs}


def write_model_dir(config, out_dir: str, seed: int = 0, std: float = 0.02,
                    norm_std: float = 0.01, dtype: torch.dtype = torch.float32) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a family's
    typed config with ``to_dict()`` and ``to_spec()``).  Returns ``out_dir``."""
    from ..parts.model import param_specs_for  # deferred: parts import weights
    os.makedirs(out_dir, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    specs = param_specs_for(config.to_spec())
    tensors = random_tensors(specs, seed, std, norm_std, dtype)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return out_dir
