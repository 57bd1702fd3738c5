"""Weights from a model folder by tensor name.

The model says which tensors it expects (name -> ``TensorSpec``); the folder is
checked against that list as a whole, and ONE error lists every missing tensor,
every unexpected one and every wrong shape.  The reference checks tensor by
tensor and stops at the first ("tensor %s missing", "tensor %s: unexpected type
or shape": src/llm/model_load.c:53-77); a tied head is an absent output matrix
(src/llm/model_load.c:1004-1007).

Resident dtypes: with compute dtype bfloat16 a tensor stored as BF16 or F16 is
kept in bfloat16, a tensor stored in 32-bit floats stays in 32-bit floats, and a
table of integers becomes int32.  With compute dtype float32 every float tensor
is widened to float32 (exactly; nothing is rounded).
"""
from __future__ import annotations

from typing import Iterator, List, Mapping, Tuple

import torch

from .safetensors_io import Checkpoint, SafetensorsError
from .spec import INT_TABLE, TensorSpec


class WeightError(ValueError):
    """The folder's tensors do not match what the model needs."""

    def __init__(self, model_dir: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_type: List[Tuple[str, str]]):
        self.missing, self.unexpected = missing, unexpected
        self.wrong_shape, self.wrong_type = wrong_shape, wrong_type
        lines = [f"{model_dir}: the weights do not match the configuration"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, want, got in wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, dt in wrong_type:
            lines.append(f"  wrong type: {name} is stored as {dt}")
        super().__init__("\n".join(lines))


_FLOATS = ("F32", "F16", "BF16")
_INTS = ("I32", "I64")


def resident_dtype(stored: str, kind: str, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device."""
    if kind == INT_TABLE:
        return torch.int32
    if compute_dtype == torch.float32 or stored == "F32":
        return torch.float32
    return torch.bfloat16


def check(ckpt: Checkpoint, expected: Mapping[str, TensorSpec]) -> None:
    missing = [n for n, s in expected.items() if n not in ckpt.tensors and not s.optional]
    unexpected = [n for n in ckpt.tensors if n not in expected]
    wrong_shape, wrong_type = [], []
    for name, spec in expected.items():
        info = ckpt.tensors.get(name)
        if info is None:
            continue
        if tuple(info.shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(spec.shape), tuple(info.shape)))
        ok = _INTS if spec.kind == INT_TABLE else _FLOATS
        if info.dtype not in ok:
            wrong_type.append((name, info.dtype))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(ckpt.model_dir, sorted(missing), sorted(unexpected),
                          wrong_shape, wrong_type)


def load_tensors(model_dir: str, expected: Mapping[str, TensorSpec],
                 compute_dtype: torch.dtype) -> Iterator[Tuple[str, torch.Tensor]]:
    """Checks the folder against ``expected`` and then yields (name, host
    tensor in its resident dtype), one tensor at a time."""
    if compute_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"compute dtype {compute_dtype}: float32 or bfloat16")
    with Checkpoint(model_dir) as ckpt:
        check(ckpt, expected)
        for name, spec in expected.items():
            info = ckpt.tensors.get(name)
            if info is None:
                continue
            t = ckpt.read(name)
            want = resident_dtype(info.dtype, spec.kind, compute_dtype)
            if spec.kind == INT_TABLE and t.dtype == torch.int64:
                if t.numel() and (int(t.max()) > 2**31 - 1 or int(t.min()) < -2**31):
                    raise SafetensorsError(f"{model_dir}: {name} does not fit int32")
            yield name, t.to(want)
