"""Random weights: a model folder made from a configuration and a seed.

Every linear and embedding weight is N(0, 0.02) and every norm weight
1 + N(0, 0.1).  Each tensor has a generator of its own, seeded from the seed
and the tensor's name, so a tensor's values do not depend on which other
tensors exist or on their order.  The reference has no such mode (its tests use
random bytes for single kernels, tests/test_cuda_kernels.c:92-118).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator, Mapping, Tuple

import torch

from .safetensors_io import write_safetensors
from .spec import EMBEDDING, INT_TABLE, MATRIX, NORM, TensorSpec

MATRIX_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & (2**63 - 1)


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: str | torch.device = "cpu") -> torch.Tensor:
    """The tensor ``name`` of the random model ``seed``, drawn in float32 on
    ``device`` and then stored as ``dtype``.  A given device type always gives
    the same values; host and GPU generators differ from each other."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.kind == INT_TABLE:
        raise ValueError(f"{name}: no random rule for integer tables")
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.kind == NORM:
        t.mul_(NORM_STD).add_(1.0)
    elif spec.kind in (MATRIX, EMBEDDING):
        t.mul_(MATRIX_STD)
    else:
        raise ValueError(f"{name}: unknown tensor kind {spec.kind}")
    return t.to(dtype)


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                   device: str | torch.device = "cpu",
                   include_optional: bool = False) -> Iterator[Tuple[str, torch.Tensor]]:
    for name, spec in expected.items():
        if spec.optional and not include_optional:
            continue
        yield name, random_tensor(name, spec, seed, dtype, device)


def write_random_model(model_dir: str, config, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` (a
    registered architecture's typed configuration) with weights from ``seed``,
    stored as ``dtype`` (bfloat16 or float32)."""
    from . import expected_tensors  # the same list the loader checks

    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("random weights are stored as bfloat16 or float32")
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    expected = expected_tensors(config.to_model_spec())
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(expected, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
