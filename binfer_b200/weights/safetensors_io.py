"""Reading and writing safetensors files, by tensor name.

Format (as the reference parses it, src/loader/safetensors.ts:32-91): an 8-byte
little-endian header length, a JSON header mapping each name to ``dtype``,
``shape`` and ``data_offsets`` relative to the end of the header, then raw
little-endian data.  ``__metadata__`` is skipped (:62).  The reference reads
only the first MiB for the header (src/loader/mmap_loader.ts:136); here the
whole file is memory-mapped, so the header may have any length.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype -> (numpy dtype used to view the bytes, bytes per element)
_NP = {
    "F64": (np.float64, 8), "F32": (np.float32, 4), "F16": (np.float16, 2),
    "BF16": (np.uint16, 2), "I64": (np.int64, 8), "I32": (np.int32, 4),
    "I16": (np.int16, 2), "I8": (np.int8, 1), "U8": (np.uint8, 1), "BOOL": (np.bool_, 1),
}
_TORCH_TO_ST = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
    torch.uint8: "U8", torch.bool: "BOOL",
}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    start: int      # absolute byte offset in the file
    end: int
    path: str


def read_header(path: str) -> Dict[str, TensorInfo]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds file size {size}")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
    base = 8 + n
    out: Dict[str, TensorInfo] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dtype = meta["dtype"]
        if dtype not in _NP:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
        shape = tuple(int(s) for s in meta["shape"])
        a, b = (int(x) for x in meta["data_offsets"])
        numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if b - a != numel * _NP[dtype][1]:
            raise SafetensorsError(
                f"{path}: tensor {name!r} spans {b - a} bytes but shape {list(shape)} of "
                f"{dtype} needs {numel * _NP[dtype][1]}")
        if base + b > size:
            raise SafetensorsError(f"{path}: tensor {name!r} reaches past the end of the file")
        out[name] = TensorInfo(name, dtype, shape, base + a, base + b, path)
    return out


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are materialised one by one."""

    def __init__(self, path: str):
        self.path = path
        self.infos = read_header(path)
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) \
            if os.path.getsize(path) else None

    def names(self) -> List[str]:
        return list(self.infos)

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor in its stored precision, except that 16-bit floats become
        bfloat16, 64-bit floats float32 and integers int32."""
        info = self.infos[name]
        np_dtype, _ = _NP[info.dtype]
        numel = int(np.prod(info.shape, dtype=np.int64)) if info.shape else 1
        arr = np.frombuffer(self._mm, dtype=np_dtype, count=numel, offset=info.start)
        arr = arr.reshape(info.shape)
        if info.dtype == "BF16":
            return torch.from_numpy(arr.copy()).view(torch.bfloat16)
        if info.dtype == "F16":
            return torch.from_numpy(arr.copy()).to(torch.bfloat16)
        if info.dtype == "F32":
            return torch.from_numpy(arr.copy())
        if info.dtype == "F64":
            return torch.from_numpy(arr.astype(np.float32))
        return torch.from_numpy(arr.astype(np.int32))

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str,
              metadata: Dict[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU or device) as one safetensors file, names sorted."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs: List[bytes] = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    js = json.dumps(header, separators=(",", ":")).encode("utf-8")
    js += b" " * (-len(js) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for b in blobs:
            f.write(b)
