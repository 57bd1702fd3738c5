"""Configuration: typed per-architecture classes, the neutral ``ModelSpec`` they
produce, and the registry that finds the class for a ``config.json``.

The reading, checking and the registry are the library's (``config/qwen3.cpp``,
``config/registry.cpp``, ``config/spec.cpp``); the classes here hold what it
returns.  A ``ModelSpec`` can also be put together by hand from ``PartSpec``s of
registered parts and opened directly (``janas_b200.engine.Engine.from_spec``).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from .. import lib


class ConfigError(ValueError):
    """A configuration that cannot be built: a missing key, a wrong value."""

    def __init__(self, message: str, code: int = lib.EOPEN):
        super().__init__(message)
        self.code = code


def _call(method: str, **args):
    try:
        return lib.call(method, **args)
    except lib.LLMError as e:
        raise ConfigError(str(e), e.code) from None


def _plain(v: Any) -> Any:
    """Parameters as JSON holds them (tuples become lists, parts become objects)."""
    if isinstance(v, PartSpec):
        return v.to_json()
    if isinstance(v, Mapping):
        return {k: _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered kind and its constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def __hash__(self) -> int:
        return hash((self.kind, json.dumps(_plain(self.params), sort_keys=True)))

    def to_json(self) -> Dict[str, Any]:
        return {"kind": self.kind, "params": _plain(self.params)}

    @staticmethod
    def from_json(d: Mapping[str, Any]) -> "PartSpec":
        params = {k: (PartSpec.from_json(v) if isinstance(v, dict) and set(v) == {"kind", "params"}
                      else v) for k, v in (d.get("params") or {}).items()}
        return PartSpec(d["kind"], params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged and where its tensors are found."""

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
    """One entry of the run order: run ``layer`` (its weights).  With ``cache_of``
    set (the index of an earlier entry) the entry's mixer writes nothing and reads
    that entry's cache."""

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

    def to_json(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture, "hidden_size": self.hidden_size,
            "vocab_size": self.vocab_size, "max_positions": self.max_positions,
            "layers": [{"block": l.block, "mixer": l.mixer.to_json(),
                        "feed_forward": l.feed_forward.to_json(),
                        "mixer_norm": l.mixer_norm.to_json(), "ffn_norm": l.ffn_norm.to_json(),
                        "prefix": l.prefix, "mixer_name": l.mixer_name, "ffn_name": l.ffn_name,
                        "mixer_norm_name": l.mixer_norm_name, "ffn_norm_name": l.ffn_norm_name}
                       for l in self.layers],
            "run_order": [{"layer": e.layer, "cache_of": e.cache_of} for e in self.run_order],
            "final_norm": self.final_norm.to_json(), "tie_embeddings": self.tie_embeddings,
            "embedding_name": self.embedding_name, "final_norm_name": self.final_norm_name,
            "head_name": self.head_name}

    @staticmethod
    def from_json(d: Mapping[str, Any]) -> "ModelSpec":
        layers = tuple(LayerSpec(
            l["block"], PartSpec.from_json(l["mixer"]), PartSpec.from_json(l["feed_forward"]),
            PartSpec.from_json(l["mixer_norm"]), PartSpec.from_json(l["ffn_norm"]), l["prefix"],
            l["mixer_name"], l["ffn_name"], l["mixer_norm_name"], l["ffn_norm_name"])
            for l in d["layers"])
        return ModelSpec(
            architecture=d["architecture"], hidden_size=d["hidden_size"],
            vocab_size=d["vocab_size"], max_positions=d["max_positions"], layers=layers,
            run_order=tuple(RunEntry(e["layer"], e["cache_of"]) for e in d["run_order"]),
            final_norm=PartSpec.from_json(d["final_norm"]), tie_embeddings=d["tie_embeddings"],
            embedding_name=d["embedding_name"], final_norm_name=d["final_norm_name"],
            head_name=d["head_name"])

    def validate(self) -> None:
        _call("spec.validate", spec=self.to_json())


@dataclass(frozen=True)
class Qwen3Config:
    """The Qwen3 dense decoder's ``config.json`` keys, as the library read them."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    layer_types: Tuple[str, ...] = ()
    sliding_window: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Qwen3ForCausalLM"
    _json: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)
    _spec: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        return _wrap(_call("config.parse", config=dict(d)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self._json)

    def to_model_spec(self) -> ModelSpec:
        return ModelSpec.from_json(self._spec)


def _wrap(r: Mapping[str, Any]):
    c = r["config"]
    n = c["num_hidden_layers"]
    if r["architecture"] != "Qwen3ForCausalLM" and c.get("model_type") != "qwen3":
        raise ConfigError(f"no Python class for architecture {r['architecture']!r}")
    return Qwen3Config(
        vocab_size=c["vocab_size"], hidden_size=c["hidden_size"],
        intermediate_size=c["intermediate_size"], num_hidden_layers=n,
        num_attention_heads=c["num_attention_heads"],
        num_key_value_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
        max_position_embeddings=c["max_position_embeddings"], rms_norm_eps=c["rms_norm_eps"],
        rope_theta=c["rope_theta"], tie_word_embeddings=c["tie_word_embeddings"],
        layer_types=tuple(c.get("layer_types") or ["full_attention"] * n),
        sliding_window=c.get("sliding_window"), eos_token_ids=tuple(r["eos_token_ids"]),
        architecture=r["architecture"], _json=c, _spec=r["spec"])


def known_architectures() -> list:
    return sorted(_call("config.known")["architectures"])


def config_from_dict(d: Mapping[str, Any]):
    """The typed configuration for a ``config.json`` given as a dictionary."""
    return _wrap(_call("config.parse", config=dict(d)))


def config_from_dir(model_dir: str):
    """The typed configuration of the model folder ``model_dir``."""
    return _wrap(_call("config.from_dir", dir=str(model_dir)))


__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
           "config_from_dict", "config_from_dir", "known_architectures"]
