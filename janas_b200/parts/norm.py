"""RMSNorm: out = (x * 1/sqrt(mean(x^2) + eps)) * w
(src/llm/model_impl.h:635-644).  The weight is used as it is, not as 1 + w."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..csrc import ops
from ..weights import NORM, TensorSpec
from .base import Norm
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: size, eps."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensors(self, prefix: str) -> Dict[str, TensorSpec]:
        return {self._name(prefix, "weight"): TensorSpec((self.size,), NORM)}

    def load(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self._name(prefix, "weight")].contiguous()

    def apply(self, x, out_dtype, delta=None, rows=None):
        if delta is not None and rows is not None:
            ops.add_(x, delta)
            delta = None
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, delta=delta, rows=rows)
