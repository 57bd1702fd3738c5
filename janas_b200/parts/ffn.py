"""The SwiGLU feed-forward: down(SiLU(gate(x)) * up(x)), no biases
(src/llm/model_ffn.c:147-154, src/llm/vmath.h:64-68).  The reference runs a
dense layer as the single expert of a mixture with router weight exactly 1
(src/llm/model_load.c:505-514); here it is a part of its own."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..csrc import ops
from ..weights import MATRIX, TensorSpec
from .base import FeedForward, StepContext
from .linear import fuse_rows, product
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size."""

    # Rows from which gate, up and the activation run as one kernel
    # (ops.linear_swiglu).  Measured on B200 at Qwen3-4B sizes: 167 against 165 + 37
    # microseconds at 2,048 rows, 103 against 109 at 1,024, even at 512; with few rows
    # the one kernel cannot cut k into parts and loses (29 against 20 at 8 rows).
    FUSED_FROM = 512
    # Rows up to which the one kernel runs too, in tiles of 64 gate and 64 up
    # features, if the plain product would not cut k either (a wide feed-forward:
    # the tiles alone fill the SMs).  It saves the activation kernel of a decode step.
    FUSED_UP_TO = 64

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensors(self, prefix: str) -> Dict[str, TensorSpec]:
        n = self._name
        return {
            n(prefix, "gate_proj.weight"): TensorSpec((self.inter, self.hidden), MATRIX),
            n(prefix, "up_proj.weight"): TensorSpec((self.inter, self.hidden), MATRIX),
            n(prefix, "down_proj.weight"): TensorSpec((self.hidden, self.inter), MATRIX),
        }

    def load(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self._name
        self.w_gate_up = fuse_rows([tensors[n(prefix, "gate_proj.weight")],
                                    tensors[n(prefix, "up_proj.weight")]])
        self.w_down = tensors[n(prefix, "down_proj.weight")].contiguous()

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        act = None
        if ctx.dtype == torch.bfloat16 and (
                ctx.n_rows >= self.FUSED_FROM or
                (ctx.n_rows <= self.FUSED_UP_TO and
                 ops.linear_parts(ctx.n_rows, 2 * self.inter, self.hidden) == 1)):
            # enough rows, or enough features, to fill the SMs without cutting k:
            # gate, up and the activation in one kernel
            act = ops.linear_swiglu(h, self.w_gate_up)
        if act is None:
            act = ops.swiglu(product(h, self.w_gate_up), ctx.dtype)
        return product(act, self.w_down)
