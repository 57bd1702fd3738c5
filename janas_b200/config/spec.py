"""Architecture-neutral description of a decoder: what the engine builds from.

A typed architecture configuration (for instance ``Qwen3Config``) is turned
into a ``ModelSpec``.  The spec is plain data: for every layer it names the
mixer, the feed-forward, the norms and the block arrangement together with
their constants, and ``run_order`` lists which layers run in which order.  The
engine, the cache and the weight loader read only this spec, never the
architecture's own configuration, so that a second architecture adds a
configuration class and a ``to_model_spec`` and nothing else.

The reference keeps the same information in a table row per architecture and
per-layer fields (``struct janas_arch`` src/llm/arch.h:21-62, ``struct layer``
src/llm/model_impl.h:36-106); layers that read another layer's keys and values
are src/llm/model_load.c:1047-1056.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built: a missing key, a wrong value."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered kind and its constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def __hash__(self) -> int:  # params may hold nested PartSpecs and tuples
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged and where its tensors are found.

    ``prefix`` is the layer's tensor-name prefix in the checkpoint and the four
    ``*_name`` fields are the sub-prefixes of its parts below it.
    """

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    prefix: str
    mixer_name: str = "self_attn"
    ffn_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    ffn_norm_name: str = "post_attention_layernorm"


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run ``layer`` (its weights).

    A layer may be named by several entries; every entry is a place of its own
    in the cache.  With ``cache_of`` set (the index of an earlier entry of the
    run order) the entry's mixer writes nothing and reads that entry's cache.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    tie_embeddings: bool
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0 or self.max_positions <= 0:
            raise ConfigError("hidden_size, vocab_size and max_positions must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not self.run_order:
            raise ConfigError("the run order is empty")
        for at, entry in enumerate(self.run_order):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"run order entry {at} names layer {entry.layer}, "
                                  f"the model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < at:
                    raise ConfigError(f"run order entry {at} reads the cache of entry "
                                      f"{entry.cache_of}, which has not run before it")
                if self.run_order[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"run order entry {at} reads the cache of entry "
                                      f"{entry.cache_of}, which owns none")
