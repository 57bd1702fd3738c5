"""NeoX ("rotate half") rotary position encoding.

theta(p, i) = (float)p * powf(theta, -2 i / rotary_dim), i < rotary_dim / 2; the
pair (i, i + half) of a head is rotated by it (src/llm/model.c:100-113,
src/llm/model_attn.c:31-39).  The powers are computed once on the host in double
and rounded to float, as the reference's powf does (src/llm/jmath.c:131-134);
the table of cos and sin is filled on the device from double-precision sincos of
the float angle (src/llm/jmath.c:163-200) when the cache's size is known.

The rotation itself is applied by the attention kernel that also normalizes the
heads and appends K and V (csrc/rope.cu); this part owns the constants and the
table.  Only the whole head can be rotated (rotary_dim == head size); the
reference's partial rotation (n_rot < head size) is not built.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..config import ConfigError
from ..csrc import ops
from .base import PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rope_neox")
class RopeNeox(PositionEncoding):
    """params: rotary_dim, theta, max_positions."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.theta = float(spec.params["theta"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ConfigError("rope_neox: rotary_dim must be even and positive")
        half = self.rotary_dim // 2
        expo = np.float32(-2.0) * np.arange(half, dtype=np.float32) / np.float32(self.rotary_dim)
        self.inv_freq_host = np.power(np.float64(np.float32(self.theta)),
                                      expo.astype(np.float64)).astype(np.float32)
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, n_positions: int) -> None:
        n = min(n_positions, self.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n:
            return
        inv = torch.from_numpy(self.inv_freq_host).to(self.device)
        self.cos, self.sin = ops.rope_table(inv, n)

    @property
    def n_positions(self) -> int:
        return 0 if self.cos is None else self.cos.shape[0]


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    """No position encoding: q and k are used as they are."""

    cos = None
    sin = None
    rotary_dim = 0
    n_positions = 1 << 62
