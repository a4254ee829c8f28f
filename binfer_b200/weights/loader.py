"""Checkpoint loading by tensor name, with one error for everything that is wrong.

The reference uploads whatever the files hold, finds a missing tensor only when
a layer first asks for it (``Weight not found``, src/engine/device_context.ts:64-67)
and checks no shape (src/loader/mmap_loader.ts:112-231).  Here the model states
up front which names and shapes it needs (:class:`ParamSpec`), and
:func:`check_names` reports missing tensors, unexpected tensors and wrong shapes
together.

File discovery follows src/loader/mmap_loader.ts:88-107: ``model.safetensors`` if
it exists, else every ``*.safetensors`` in the folder, sorted.  Unlike the
reference, ``model.safetensors.index.json`` is read when it is there: the model is
then exactly the shards that its ``weight_map`` names; a shard that is missing is
one error that names it, and a ``*.safetensors`` file that the index does not
name is left alone, with a warning.
"""
from __future__ import annotations

import json
import os
import warnings
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile


@dataclass(frozen=True)
class ParamSpec:
    """One tensor that a part needs from the checkpoint."""

    name: str
    shape: Tuple[int, ...]
    # how the random-weights mode fills it: "matrix" ~ N(0, s), "norm" ~ 1 + N(0, s_norm)
    init: str = "matrix"
    # a matrix feeds a matrix product and takes the engine's compute dtype;
    # a vector (norm weight, bias) is held in 32-bit whatever it was stored in
    role: str = "matrix"


class WeightError(ValueError):
    """Raised once, listing every missing, unexpected and wrongly shaped tensor."""

    def __init__(self, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]], where: str = ""):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"checkpoint {where} does not match the model:".replace("  ", " ")]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        super().__init__("\n".join(lines))


INDEX_FILE = "model.safetensors.index.json"


def read_index(model_dir: str) -> Optional[Dict[str, str]]:
    """``weight_map`` (tensor name -> shard file) of the folder's index, or None without one."""
    path = os.path.join(model_dir, INDEX_FILE)
    if not os.path.exists(path):
        return None
    with open(path) as f:
        index = json.load(f)
    wm = index.get("weight_map")
    if not isinstance(wm, dict) or not wm:
        raise ValueError(f"{path} has no weight_map")
    return {str(k): str(v) for k, v in wm.items()}


def find_safetensors_files(model_dir: str) -> List[str]:
    """The files that hold the model.  With an index: its shards, all of which must exist
    (one error names every missing one); files the index does not name are ignored, with a
    warning.  Without: ``model.safetensors``, else every ``*.safetensors``, sorted."""
    present = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    index = read_index(model_dir)
    if index is not None:
        shards = sorted(set(index.values()))
        gone = [f for f in shards if not os.path.exists(os.path.join(model_dir, f))]
        if gone:
            raise FileNotFoundError(
                f"{model_dir}: {INDEX_FILE} names shards that are not there "
                f"({len(gone)} of {len(shards)}): " + ", ".join(gone))
        extra = [f for f in present if f not in shards]
        if extra:
            warnings.warn(f"{model_dir}: ignoring safetensors files that {INDEX_FILE} does not "
                          f"name: " + ", ".join(extra))
        return [os.path.join(model_dir, f) for f in shards]
    if "model.safetensors" in present:
        return [os.path.join(model_dir, "model.safetensors")]
    if not present:
        raise FileNotFoundError(f"No safetensors files found in {model_dir}")
    return [os.path.join(model_dir, f) for f in present]


def check_names(specs: Iterable[ParamSpec], found: Mapping[str, Tuple[int, ...]],
                optional: Iterable[str] = (), where: str = "",
                allow_unexpected: bool = False) -> None:
    """Raise :class:`WeightError` unless ``found`` (name -> shape) is exactly ``specs``.

    Names in ``optional`` may be present without being asked for (a stored
    ``lm_head.weight`` beside tied embeddings, for instance).  With
    ``allow_unexpected`` tensors that nobody asked for are named in a warning instead
    of the error (the reference uploads them silently, src/loader/mmap_loader.ts:175-225);
    missing tensors and wrong shapes are an error either way.
    """
    want = {s.name: tuple(s.shape) for s in specs}
    optional = set(optional)
    missing = sorted(n for n in want if n not in found)
    unexpected = sorted(n for n in found if n not in want and n not in optional)
    wrong = sorted((n, tuple(found[n]), want[n]) for n in want
                   if n in found and tuple(found[n]) != want[n])
    if allow_unexpected and unexpected and not (missing or wrong):
        warnings.warn(f"checkpoint {where}: ignoring {len(unexpected)} tensors the model does "
                      f"not use: " + ", ".join(unexpected[:20])
                      + (" ..." if len(unexpected) > 20 else ""))
        return
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)


class Checkpoint:
    """All safetensors files of a model folder, addressed by tensor name."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files = [SafetensorsFile(p) for p in find_safetensors_files(model_dir)]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self._where[n] = f
        index = read_index(model_dir)
        if index is not None:
            # the index is the model's own list: a tensor it names must be in the shard it names
            by_path = {os.path.basename(f.path): f for f in self.files}
            lost = sorted(n for n, shard in index.items() if n not in by_path[shard].infos)
            if lost:
                raise WeightError(lost, [], [], where=f"{model_dir} (tensors that {INDEX_FILE} "
                                                     f"names are not in their shards)")

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: f.infos[n].shape for n, f in self._where.items()}

    def stored_dtypes(self) -> Dict[str, str]:
        return {n: f.infos[n].dtype for n, f in self._where.items()}

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


class TensorSource:
    """What a model loads from: name -> tensor, from a folder or from memory.

    ``get(name)`` returns the tensor in its stored precision (bfloat16, float32
    or int32) on whatever device it lives; the model moves and casts it.
    """

    def __init__(self, get: Callable[[str], torch.Tensor],
                 shapes: Mapping[str, Tuple[int, ...]], where: str = ""):
        self.get, self.shapes, self.where = get, dict(shapes), where

    @classmethod
    def from_dir(cls, model_dir: str) -> "TensorSource":
        ck = Checkpoint(model_dir)
        src = cls(ck.tensor, ck.shapes(), where=model_dir)
        src._checkpoint = ck
        return src

    @classmethod
    def from_dict(cls, tensors: Mapping[str, torch.Tensor], where: str = "(in memory)"):
        return cls(lambda n: tensors[n], {n: tuple(t.shape) for n, t in tensors.items()}, where)

    def close(self) -> None:
        ck = getattr(self, "_checkpoint", None)
        if ck is not None:
            ck.close()


def place(t: torch.Tensor, spec: ParamSpec, compute_dtype: torch.dtype,
          device: torch.device) -> torch.Tensor:
    """Move a stored tensor to the device in the precision its role asks for.

    Matrices take the compute dtype (bfloat16 stays bfloat16 in a bfloat16
    engine; a float32 engine widens them, which is exact).  Vectors are held in
    float32: a tensor stored in 32-bit is never narrowed, and widening a 16-bit
    one is exact.  Integer tables stay int32.
    """
    if not t.dtype.is_floating_point:
        return t.to(device=device, dtype=torch.int32).contiguous()
    dtype = torch.float32 if spec.role == "vector" else compute_dtype
    return t.to(device=device, dtype=dtype).contiguous()
