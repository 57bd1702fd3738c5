"""A weight matrix [out_features, in_features] and its product y = W x
(the reference's layout: src/llm/model_load.c:452)."""
from __future__ import annotations

from typing import Sequence

import torch

from ..csrc import ops


def fuse_rows(mats: Sequence[torch.Tensor]) -> torch.Tensor:
    """Several matrices over the same input as one, rows one after the other,
    so that one product serves them all (the reference dispatches q, k, v as one
    group and gate, up as one: src/llm/model_attn.c:255, src/llm/model_ffn.c:349).
    If their dtypes differ, the widest is taken."""
    dt = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
    return torch.cat([m.to(dt) for m in mats], dim=0).contiguous()


def product(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """a [n, in] . weight^T -> stack [S, n, out] of float32 partial sums."""
    return ops.linear(a, weight)
