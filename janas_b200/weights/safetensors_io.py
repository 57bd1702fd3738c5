"""Writing safetensors files (for the random-weights mode and for tests).

The format: an 8-byte little-endian header length, a JSON header that gives
each tensor's dtype, shape and byte range relative to the end of the header,
then the bytes.  Reading is the library's (``weights/safetensors.cpp``): the
engine maps the files and checks every field against them.
"""
from __future__ import annotations

import json
import os
import struct
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
