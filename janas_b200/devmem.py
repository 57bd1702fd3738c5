"""Device memory that the library owns, seen as PyTorch tensors (no copy).

For tests and tools that want to look at, or write into, what the engine holds:
cache pages, a mixer's per-sequence state, the arguments a registered part is
called with.  PyTorch is imported only when one of these functions is used.
"""
from __future__ import annotations

from typing import Sequence

_TYPESTR = {"float32": "<f4", "int32": "<i4", "int64": "<i8", "bfloat16": "<i2", "float16": "<f2"}


class _Memory:
    def __init__(self, ptr: int, shape: Sequence[int], typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": typestr,
                                         "data": (int(ptr), False), "version": 2}


def as_tensor(ptr: int, shape: Sequence[int], dtype: str, device: int = 0):
    """The device memory at ``ptr`` as a tensor of ``shape`` and ``dtype`` (a name:
    float32, bfloat16, int32, int64).  The tensor does not own the memory."""
    import torch
    n = 1
    for s in shape:
        n *= int(s)
    if n == 0 or not ptr:
        return torch.empty(tuple(shape), dtype=getattr(torch, dtype), device=f"cuda:{device}")
    t = torch.as_tensor(_Memory(ptr, shape, _TYPESTR[dtype]), device=f"cuda:{device}")
    return t.view(torch.bfloat16) if dtype == "bfloat16" else t


def dtype_name(dtype) -> str:
    """"float32" / "bfloat16" / ... for a torch dtype or a name."""
    s = str(dtype)
    s = s.split(".")[-1]
    return {"bf16": "bfloat16", "fp32": "float32"}.get(s, s)
