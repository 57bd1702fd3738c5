"""Registries of part kinds: one name -> class table for each role.

A new mixer, feed-forward, norm, position encoding or block arrangement is a
class registered here under a new name; a configuration then refers to it by
that name in a ``PartSpec``.  Nothing else in the framework has to change.
"""
from __future__ import annotations

from typing import Callable, Dict

import torch

from ..config import ConfigError, PartSpec

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}

_ROLES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS,
          "position": POSITION_ENCODINGS, "block": BLOCKS}


def _register(table: Dict[str, type], kind: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        table[kind] = cls
        return cls
    return deco


def register_mixer(kind: str): return _register(MIXERS, kind)
def register_feed_forward(kind: str): return _register(FEED_FORWARDS, kind)
def register_norm(kind: str): return _register(NORMS, kind)
def register_position_encoding(kind: str): return _register(POSITION_ENCODINGS, kind)
def register_block(kind: str): return _register(BLOCKS, kind)


def build_part(role: str, spec: PartSpec, dtype: torch.dtype, device: torch.device):
    table = _ROLES[role]
    cls = table.get(spec.kind)
    if cls is None:
        raise ConfigError(f"no {role} of kind {spec.kind!r}; registered: "
                          + ", ".join(sorted(table)))
    return cls(spec, dtype, device)


def block_class(kind: str) -> type:
    cls = BLOCKS.get(kind)
    if cls is None:
        raise ConfigError(f"no block arrangement {kind!r}; registered: "
                          + ", ".join(sorted(BLOCKS)))
    return cls
