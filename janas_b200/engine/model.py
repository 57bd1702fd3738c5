"""The one generic decoder: embedding, the layers in run order, final norm, head.

It is built from a ``ModelSpec`` alone.  For every layer the spec names the
block arrangement, the mixer, the feed-forward and the norms; the classes come
from the part registries.  ``run_order`` is walked entry by entry; an entry
names the layer whose weights run and, optionally, an earlier entry whose cache
it reads instead of writing one of its own.

The reference's forward pass has the same shape: embedding, layer loop, final
norm of the rows whose logits are wanted, head (src/llm/model.c:647-876; the
head is the embedding table when the file has no output matrix:
src/llm/model_load.c:1004-1007).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..cache import KVSpec, StateSpec
from ..config import ModelSpec
from ..csrc import ops
from ..parts import Block, LayerCache, StepContext, block_class, build_part
from ..weights import EMBEDDING, MATRIX, TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the compute dtype is float32 or bfloat16")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks: List[Block] = []
        for ls in spec.layers:
            cls = block_class(ls.block)
            self.blocks.append(cls(
                build_part("mixer", ls.mixer, dtype, self.device),
                build_part("feed_forward", ls.feed_forward, dtype, self.device),
                build_part("norm", ls.mixer_norm, dtype, self.device),
                build_part("norm", ls.ffn_norm, dtype, self.device)))
        self.final_norm = build_part("norm", spec.final_norm, dtype, self.device)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # -------------------------------------------------------------- weights
    def _layer_names(self, i: int) -> Tuple[str, str, str, str]:
        ls = self.spec.layers[i]
        return (f"{ls.prefix}.{ls.mixer_name}", f"{ls.prefix}.{ls.ffn_name}",
                f"{ls.prefix}.{ls.mixer_norm_name}", f"{ls.prefix}.{ls.ffn_norm_name}")

    def tensors(self) -> Dict[str, TensorSpec]:
        """Every tensor the model reads, by checkpoint name."""
        s = self.spec
        t: Dict[str, TensorSpec] = {
            s.embedding_name: TensorSpec((s.vocab_size, s.hidden_size), EMBEDDING)}
        for i, b in enumerate(self.blocks):
            mixer, ffn, n1, n2 = self._layer_names(i)
            t.update(b.mixer_norm.tensors(n1))
            t.update(b.mixer.tensors(mixer))
            t.update(b.ffn_norm.tensors(n2))
            t.update(b.feed_forward.tensors(ffn))
        t.update(self.final_norm.tensors(s.final_norm_name))
        t[s.head_name] = TensorSpec((s.vocab_size, s.hidden_size), MATRIX,
                                    optional=s.tie_embeddings)
        return t

    def load(self, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
        """Takes (name, tensor) pairs in their resident dtype, moves them to the
        device and hands them to the parts."""
        have: Dict[str, torch.Tensor] = {}
        for name, t in tensors:
            have[name] = t.to(self.device, non_blocking=True)
        s = self.spec
        self.embedding = have[s.embedding_name].contiguous()
        if s.head_name in have:
            self.head = have[s.head_name].contiguous()
        elif s.tie_embeddings:
            self.head = self.embedding
        else:
            raise KeyError(s.head_name)
        for i, b in enumerate(self.blocks):
            mixer, ffn, n1, n2 = self._layer_names(i)
            b.mixer_norm.load(n1, have)
            b.mixer.load(mixer, have)
            b.ffn_norm.load(n2, have)
            b.feed_forward.load(ffn, have)
        self.final_norm.load(s.final_norm_name, have)

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads once (the embedding table counts only
        as the head, when tied; else only a few rows of it are read)."""
        seen, total = set(), 0

        def add(t: Optional[torch.Tensor]) -> None:
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        add(self.head)
        for b in self.blocks:
            for part in (b.mixer, b.feed_forward, b.mixer_norm, b.ffn_norm):
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
        return total

    # ---------------------------------------------------------------- cache
    def kv_specs(self) -> List[Optional[KVSpec]]:
        """Per run-order entry: what the cache holds for it."""
        return [None if e.cache_of is not None else self.blocks[e.layer].mixer.kv_spec()
                for e in self.spec.run_order]

    def state_specs(self) -> List[Optional[StateSpec]]:
        return [self.blocks[e.layer].mixer.state_spec() for e in self.spec.run_order]

    def prepare(self, n_positions: int) -> None:
        for b in self.blocks:
            b.mixer.prepare(n_positions)

    def supports(self, kind: str) -> bool:
        return all(b.mixer.supports(kind) for b in self.blocks)

    # -------------------------------------------------------------- forward
    def forward(self, ctx: StepContext, tokens: torch.Tensor, caches: Sequence[LayerCache],
                want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """tokens: int32 [n] on the device; caches[e]: the cache view of
        run-order entry e; want_rows: int32 row indices whose logits are wanted
        (None: all rows; empty: none).  Returns float32 [wanted, vocab]."""
        x = ops.embed(self.embedding, tokens)
        pending = None
        for e, entry in enumerate(self.spec.run_order):
            x, pending = self.blocks[entry.layer].forward(ctx, x, pending, caches[e])
        if want_rows is not None and want_rows.numel() == 0:
            return None
        h = self.final_norm.apply(x, ctx.dtype, delta=pending, rows=want_rows)
        return ops.linear(h, self.head, whole=True)[0]


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """The tensor list of a model of this spec (no device memory is touched)."""
    return DecoderModel(spec, torch.float32, "cpu").tensors()
