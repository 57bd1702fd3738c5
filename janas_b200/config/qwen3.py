"""Typed configuration of the Qwen3 dense decoder, read from its ``config.json``.

The keys are the architecture's own (the ones the reference's converter reads
for a Hugging Face model folder, tools/hf2gguf.c:245-277, and the
hyper-parameters its loader requires, src/llm/model_load.c:817-836).  No size
has a default in code except where the reference has one: ``head_dim`` falls
back to ``hidden_size / num_attention_heads`` (tools/hf2gguf.c:262-263) and
``tie_word_embeddings`` to false (tools/hf2gguf.c:264-265).

What Qwen3 dense does not have is refused here instead of being ignored:
attention biases, RoPE scaling, an activation other than SiLU (the reference's
table row for ``qwen3`` sets no flag: src/llm/arch.c:11).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

_REQUIRED = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
    "rms_norm_eps", "rope_theta",
)

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


def _as_int(d: Mapping[str, Any], key: str) -> int:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: {key} must be a whole number, got {v!r}")
    return int(v)


def _as_float(d: Mapping[str, Any], key: str) -> float:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Qwen3Config:
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
    # layer_types[i] is "full_attention" or "sliding_attention"; a sliding
    # layer sees the last ``sliding_window`` positions, itself included
    # (src/llm/attention.c:736-739).
    layer_types: Tuple[str, ...] = ()
    sliding_window: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Qwen3ForCausalLM"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ read
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d or d[k] is None]
        if missing:
            raise ConfigError("config.json: missing " + ", ".join(missing))
        hidden = _as_int(d, "hidden_size")
        heads = _as_int(d, "num_attention_heads")
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive")
        if d.get("head_dim") is not None:
            head_dim = _as_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError("config.json: no head_dim, and hidden_size is not a "
                                  "multiple of num_attention_heads")
            head_dim = hidden // heads
        if d.get("attention_bias"):
            raise ConfigError("config.json: attention_bias is set; the Qwen3 dense decoder "
                              "has no attention biases")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is set; only plain RoPE is built")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r}; Qwen3 uses silu")
        n_layers = _as_int(d, "num_hidden_layers")

        window = None
        layer_types: Tuple[str, ...]
        use_window = bool(d.get("use_sliding_window", False))
        if d.get("layer_types") is not None:
            layer_types = tuple(d["layer_types"])
            if len(layer_types) != n_layers:
                raise ConfigError(f"config.json: layer_types has {len(layer_types)} entries "
                                  f"for {n_layers} layers")
            bad = [t for t in layer_types if t not in (FULL_ATTENTION, SLIDING_ATTENTION)]
            if bad:
                raise ConfigError(f"config.json: unknown layer type {bad[0]!r}")
        elif use_window:
            first = _as_int(d, "max_window_layers") if d.get("max_window_layers") is not None else 0
            layer_types = tuple(SLIDING_ATTENTION if i >= first else FULL_ATTENTION
                                for i in range(n_layers))
        else:
            layer_types = (FULL_ATTENTION,) * n_layers
        if SLIDING_ATTENTION in layer_types:
            if d.get("sliding_window") is None:
                raise ConfigError("config.json: sliding layers but no sliding_window")
            window = _as_int(d, "sliding_window")
            if window <= 0:
                raise ConfigError("config.json: sliding_window must be positive")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)

        archs = d.get("architectures") or ["Qwen3ForCausalLM"]
        known = set(_REQUIRED) | {
            "head_dim", "attention_bias", "rope_scaling", "hidden_act", "use_sliding_window",
            "layer_types", "max_window_layers", "sliding_window", "eos_token_id",
            "architectures", "tie_word_embeddings"}
        cfg = cls(
            vocab_size=_as_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_as_int(d, "intermediate_size"),
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=_as_int(d, "num_key_value_heads"),
            head_dim=head_dim,
            max_position_embeddings=_as_int(d, "max_position_embeddings"),
            rms_norm_eps=_as_float(d, "rms_norm_eps"),
            rope_theta=_as_float(d, "rope_theta"),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            layer_types=layer_types,
            sliding_window=window,
            eos_token_ids=eos_ids,
            architecture=str(archs[0]),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    # ----------------------------------------------------------------- check
    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive")
        # src/llm/model_load.c:827 (heads a multiple of KV heads)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("config.json: num_attention_heads must be a multiple of "
                              "num_key_value_heads")
        if self.head_dim % 2:
            raise ConfigError("config.json: head_dim must be even (RoPE rotates pairs)")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("config.json: rope_theta must be positive")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError("layer_types must name every layer")

    # ----------------------------------------------------------------- write
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "attention_bias": False,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if SLIDING_ATTENTION in self.layer_types:
            d["use_sliding_window"] = True
            d["sliding_window"] = self.sliding_window
            d["layer_types"] = list(self.layer_types)
        else:
            d["use_sliding_window"] = False
            d["sliding_window"] = None
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d

    # ------------------------------------------------------------ the layers
    def to_model_spec(self) -> ModelSpec:
        """The decoder as parts: pre-norm blocks of GQA attention (per-head
        q/k RMSNorm, NeoX RoPE over the whole head) and a SwiGLU feed-forward,
        all RMSNorm with one eps (src/llm/model.c:743-796,
        src/llm/model_attn.c:93-101)."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rope_neox", {"rotary_dim": self.head_dim, "theta": self.rope_theta,
                                      "max_positions": self.max_position_embeddings})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                  "intermediate_size": self.intermediate_size})
        layers = []
        for i, kind in enumerate(self.layer_types):
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qk_norm_eps": self.rms_norm_eps,
                "window": self.sliding_window if kind == SLIDING_ATTENTION else 0,
                "position": rope,
            })
            layers.append(LayerSpec(block="prenorm", mixer=mixer, feed_forward=ffn,
                                    mixer_norm=norm, ffn_norm=norm,
                                    prefix=f"model.layers.{i}"))
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            layers=tuple(layers),
            run_order=tuple(RunEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=norm,
            tie_embeddings=self.tie_word_embeddings,
        )
        spec.validate()
        return spec
