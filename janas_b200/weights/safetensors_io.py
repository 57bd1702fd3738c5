"""Reading and writing safetensors files, without a library.

The format: an 8-byte little-endian header length, a JSON header that gives
each tensor's dtype, shape and byte range relative to the end of the header,
then the bytes.  Every field is checked against the file before it is used, as
the reference's reader does (src/common/hf_safetensors.h:1-52,
tools/hf2gguf.c:117-164).  A folder may hold one ``model.safetensors`` or the
shards named by ``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file."""


# dtype name -> (bytes per element, numpy storage type, torch type)
_DTYPES = {
    "F32": (4, np.dtype("<f4"), torch.float32),
    "F16": (2, np.dtype("<f2"), torch.float16),
    "BF16": (2, np.dtype("<u2"), torch.bfloat16),
    "I32": (4, np.dtype("<i4"), torch.int32),
    "I64": (8, np.dtype("<i8"), torch.int64),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.int32: "I32", torch.int64: "I64"}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str               # "F32", "BF16", ...
    shape: Tuple[int, ...]
    begin: int               # byte range in the file
    end: int
    path: str


class SafetensorsFile:
    """One open file; tensors are read on demand from a memory map."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError as e:
            raise SafetensorsError(f"{path}: {e.strerror}") from None
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen < 2 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file "
                                   f"({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: the header is not a JSON object")
        data_start = 8 + hlen
        self.tensors: Dict[str, TensorInfo] = {}
        for name, ent in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = ent["dtype"]
                shape = tuple(int(s) for s in ent["shape"])
                b, e = (int(x) for x in ent["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for {name}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has dtype {dtype}, "
                                       f"which is not read (F32, F16, BF16, I32, I64)")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if any(s < 0 for s in shape) or b < 0 or e < b \
                    or e - b != count * _DTYPES[dtype][0] or data_start + e > size:
                raise SafetensorsError(f"{path}: tensor {name}: its byte range "
                                       f"[{b}, {e}) does not match shape {list(shape)} "
                                       f"{dtype} or lies outside the file")
            self.tensors[name] = TensorInfo(name, dtype, shape, data_start + b,
                                            data_start + e, path)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def read(self, name: str) -> torch.Tensor:
        """A copy of the tensor in host memory, in the dtype it is stored in."""
        info = self.tensors[name]
        _, npdt, tdt = _DTYPES[info.dtype]
        count = int(np.prod(info.shape, dtype=np.int64)) if info.shape else 1
        arr = np.frombuffer(self._map, dtype=npdt, count=count, offset=info.begin).copy()
        t = torch.from_numpy(arr)
        if info.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(info.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._f.close()


class Checkpoint:
    """All tensors of a model folder by name, whichever file holds them."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: no weight_map") from None
            for fname in sorted(set(weight_map.values())):
                self._open(os.path.join(model_dir, fname))
            for name, fname in weight_map.items():
                if name not in self._files[os.path.join(model_dir, fname)].tensors:
                    raise SafetensorsError(f"{index}: {name} is not in {fname}")
        elif os.path.isfile(single):
            self._open(single)
        else:
            raise SafetensorsError(f"{model_dir}: no model.safetensors "
                                   f"(nor model.safetensors.index.json)")

    def _open(self, path: str) -> None:
        f = SafetensorsFile(path)
        self._files[path] = f
        for name, info in f.tensors.items():
            if name in self.tensors:
                raise SafetensorsError(f"{path}: tensor {name} is also in "
                                       f"{self.tensors[name].path}")
            self.tensors[name] = info

    def names(self) -> List[str]:
        return list(self.tensors)

    def read(self, name: str) -> torch.Tensor:
        return self._files[self.tensors[name].path].read(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()
        self._files = {}

    def __enter__(self) -> "Checkpoint":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Writes ``tensors`` (name, host tensor) to ``path``.

    The tensors are taken one at a time, so a generator keeps only one of them
    alive; their bytes go to a temporary file first because the header, which
    comes first in the format, needs every range."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    tmp = path + ".data.tmp"
    at = 0
    with open(tmp, "wb") as data:
        for name, t in tensors:
            if t.dtype not in _NAMES:
                raise SafetensorsError(f"tensor {name}: dtype {t.dtype} is not written")
            t = t.detach().cpu().contiguous()
            raw = t.view(torch.uint16) if t.dtype == torch.bfloat16 else t
            buf = raw.numpy().tobytes()
            header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                            "data_offsets": [at, at + len(buf)]}
            data.write(buf)
            at += len(buf)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as out, open(tmp, "rb") as data:
        out.write(struct.pack("<Q", len(hj)))
        out.write(hj)
        while True:
            chunk = data.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    os.remove(tmp)
