"""Grouped-query attention with optional per-head q/k RMSNorm, a position
encoding and an optional sliding window.

In order: q, k, v products without biases; per head, RMSNorm of q and of k with
one weight vector for all heads, before the rotation; the rotation; K and V into
the cache at the row's position; causal attention, head h reading KV head
h / (heads / kv_heads), scores scaled by 1/sqrt(head size); the output product
(src/llm/model_attn.c:75-146,224-285; src/llm/attention.c:874-875,1012).  With a
window w a token at position p sees positions p + 1 - w .. p
(src/llm/attention.c:736-739).
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from ..cache import KVSpec
from ..config import ConfigError
from ..csrc import ops
from ..weights import MATRIX, NORM, TensorSpec
from .base import DECODE, LayerCache, Mixer, StepContext
from .linear import fuse_rows, product
from .registry import build_part, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (None: no
    q/k norm), window (0: none), position (a PartSpec)."""

    # everything that changes from step to step is read from device arrays, so a
    # captured decode step can be replayed
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.qk_eps = p.get("qk_norm_eps")
        self.window = int(p.get("window") or 0)
        if self.nh % self.nkv:
            raise ConfigError("gqa_attention: num_heads must be a multiple of num_kv_heads")
        if self.hd % 16 or not 16 <= self.hd <= 512:
            raise ConfigError(f"gqa_attention: head_dim {self.hd}: the kernels take head "
                              f"sizes from 16 to 512 in steps of 16")
        self.position = build_part("position", p["position"], dtype, device)
        if self.position.rotary_dim not in (0, self.hd):
            raise ConfigError("gqa_attention: only the whole head can be rotated "
                              f"(rotary_dim {self.position.rotary_dim}, head_dim {self.hd})")
        self.scale = 1.0 / math.sqrt(self.hd)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None
        self.chunk = None

    # ------------------------------------------------------------- weights
    def tensors(self, prefix: str) -> Dict[str, TensorSpec]:
        n = self._name
        t = {
            n(prefix, "q_proj.weight"): TensorSpec((self.nh * self.hd, self.hidden), MATRIX),
            n(prefix, "k_proj.weight"): TensorSpec((self.nkv * self.hd, self.hidden), MATRIX),
            n(prefix, "v_proj.weight"): TensorSpec((self.nkv * self.hd, self.hidden), MATRIX),
            n(prefix, "o_proj.weight"): TensorSpec((self.hidden, self.nh * self.hd), MATRIX),
        }
        if self.qk_eps is not None:
            t[n(prefix, "q_norm.weight")] = TensorSpec((self.hd,), NORM)
            t[n(prefix, "k_norm.weight")] = TensorSpec((self.hd,), NORM)
        return t

    def load(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self._name
        self.w_qkv = fuse_rows([tensors[n(prefix, f"{x}_proj.weight")] for x in "qkv"])
        self.w_o = tensors[n(prefix, "o_proj.weight")].contiguous()
        if self.qk_eps is not None:
            qn, kn = tensors[n(prefix, "q_norm.weight")], tensors[n(prefix, "k_norm.weight")]
            if qn.dtype != kn.dtype:
                qn, kn = qn.float(), kn.float()
            self.q_norm, self.k_norm = qn.contiguous(), kn.contiguous()

    # --------------------------------------------------------------- cache
    def kv_spec(self) -> Optional[KVSpec]:
        return KVSpec(self.nkv, self.hd, self.window)

    def prepare(self, n_positions: int) -> None:
        self.position.prepare(n_positions)
        self.chunk = ops.attention_chunk()

    def supports(self, kind: str) -> bool:
        # Every kind of step, with a window too: the pages a window group gives back
        # after a step are those that the sequence's NEXT token cannot see, and
        # tokens appended later see no further back than that one.
        return True

    # ------------------------------------------------------------- forward
    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        if ctx.max_pos >= self.position.n_positions:
            raise ValueError(f"position {ctx.max_pos} is beyond the {self.position.n_positions} "
                             f"positions the encoding was prepared for")
        qkv = product(h, self.w_qkv)
        max_chunks = ctx.max_pos // self.chunk + 1
        if self.window:
            max_chunks = min(max_chunks, (self.window - 1) // self.chunk + 2)
        if ctx.kind == DECODE and ctx.dtype == torch.bfloat16:
            # one new token per sequence: the attention kernel makes q and the new
            # key and value from the product's sums itself, where it takes the sizes
            a = ops.attention_decode_qkv(
                qkv, self.q_norm, self.k_norm, float(self.qk_eps or 0.0), self.position.cos,
                self.position.sin, cache.k, cache.v, cache.writes, ctx.row_pos, ctx.row_seq,
                cache.block_table, self.window, self.scale, max_chunks, self.nh)
            if a is not None:
                return product(a.view(ctx.n_rows, self.nh * self.hd), self.w_o)
        q = ops.qk_norm_rope_append(
            qkv, self.q_norm, self.k_norm, float(self.qk_eps or 0.0), self.position.cos,
            self.position.sin, ctx.row_pos, ctx.row_seq, cache.block_table,
            cache.k if cache.writes else None, cache.v if cache.writes else None,
            self.nh, self.nkv, self.hd, ctx.dtype)
        decode = ctx.kind == DECODE
        blocks = None
        if not decode and ctx.dtype == torch.bfloat16 and self.hd in (64, 128):
            # runs of consecutive positions, for the tensor-core kernel; the same
            # for every layer of the step with this grouping of heads
            per = ops.attention_block_positions(self.nh, self.nkv)
            blocks = ctx.extras.get(("attention_blocks", per))
            if blocks is None:
                blocks = ops.attention_blocks(ctx.seq_row0[:-1], ctx.seq_pos0, ctx.seq_len, per,
                                              ctx.device)
                ctx.extras[("attention_blocks", per)] = blocks
        a = ops.attention(q, cache.k, cache.v, ctx.row_pos, ctx.row_seq, cache.block_table,
                          self.window, self.scale, max_chunks, blocks=blocks, decode=decode)
        return product(a.view(ctx.n_rows, self.nh * self.hd), self.w_o)
