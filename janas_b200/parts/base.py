"""The interfaces of the parts a layer is put together from.

A part is built from a ``PartSpec`` (its registered kind and its constants), the
compute dtype and the device.  It says which tensors it needs below a name
prefix (``tensors``), takes them (``load``) and computes (``apply`` /
``forward``).  No part knows which model it is in: sizes and constants arrive
as parameters, everything about the current step arrives in a ``StepContext``.

Outputs of mixers and feed-forwards are *stacks of partial sums*: a float32
tensor ``[S, n, hidden]`` whose sum over S is the part's output (S = 1 unless a
matrix product was split over its inner dimension).  The block adds them to the
residual stream in the order 0 .. S-1.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

import numpy as np
import torch

from ..cache import KVSpec, StateSpec
from ..config import PartSpec
from ..weights import TensorSpec

PREFILL = "prefill"   # every sequence starts at its first token
DECODE = "decode"     # every sequence goes on by one token
EXTEND = "extend"     # anything else (tokens appended to sequences that have some)


@dataclass
class LayerCache:
    """What a mixer sees of the cache for the run-order entry it runs as."""

    k: Optional[torch.Tensor] = None            # [pages, kv_heads, PAGE, head_dim]
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None  # int32 [sequences of the step, P]
    writes: bool = True                         # False: read another entry's cache only
    state: Optional[torch.Tensor] = None        # [slots, *state shape], indexed by slot


@dataclass
class StepContext:
    """One step: the rows (tokens) it runs and where each belongs.

    Rows are the sequences' tokens one sequence after the other.  The ``row_*``
    and ``seq_slot_dev`` tensors are on the device (int32); the ``seq_*`` arrays
    are on the host."""

    kind: str
    dtype: torch.dtype
    device: torch.device
    n_rows: int
    n_seqs: int
    row_pos: torch.Tensor          # position of each row in its sequence
    row_seq: torch.Tensor          # index of the row's sequence within the step
    seq_slot_dev: torch.Tensor     # slot of each sequence
    seq_slots: List[int]
    seq_pos0: np.ndarray           # tokens each sequence had before the step
    seq_len: np.ndarray            # tokens each sequence brings
    seq_row0: np.ndarray           # first row of each sequence (len n_seqs + 1)
    max_pos: int                   # the largest position of any row
    extras: Dict[str, object] = field(default_factory=dict)


class Part:
    """Base of all parts."""

    def __init__(self, spec: PartSpec, dtype: torch.dtype, device: torch.device):
        self.spec = spec
        self.dtype = dtype
        self.device = device

    def tensors(self, prefix: str) -> Dict[str, TensorSpec]:
        """name -> TensorSpec of every tensor this part reads, below ``prefix``
        (which ends without a dot; an empty prefix means no prefix)."""
        return {}

    def load(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        """Takes its tensors (already on the device, in their resident dtype)."""

    @staticmethod
    def _name(prefix: str, leaf: str) -> str:
        return f"{prefix}.{leaf}" if prefix else leaf


class Norm(Part):
    def apply(self, x: torch.Tensor, out_dtype: torch.dtype,
              delta: Optional[torch.Tensor] = None,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normalizes the rows of the float32 residual stream ``x``.  With
        ``delta`` (a stack of partial sums) x += sum(delta) happens first, in
        place.  With ``rows`` only those rows are normalized and returned."""
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, n_positions: int) -> None:
        """Called once the cache's size is known: positions below
        ``n_positions`` will be asked for."""


class Mixer(Part):
    # True when forward() reads everything that changes between decode steps
    # (positions, slots, block tables) from the context's device arrays only, so
    # that a captured decode step can be replayed with new contents
    graph_safe = False

    def kv_spec(self) -> Optional[KVSpec]:
        """Keys and values per position that the cache should hold, or None."""
        return None

    def state_spec(self) -> Optional[StateSpec]:
        """Fixed-size state per sequence, or None."""
        return None

    def prepare(self, n_positions: int) -> None:
        pass

    def supports(self, kind: str) -> bool:
        """Whether the mixer can run a step of this kind."""
        return True

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        """h: [n, hidden] in the compute dtype -> stack [S, n, hidden] float32."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        """h: [n, hidden] in the compute dtype -> stack [S, n, hidden] float32."""
        raise NotImplementedError


class Block:
    """The arrangement of one layer's parts around the residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 ffn_norm: Norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def forward(self, ctx: StepContext, x: torch.Tensor, pending: Optional[torch.Tensor],
                cache: LayerCache):
        """x: float32 residual stream, updated in place; ``pending``: a stack
        of partial sums not yet added to x (or None).  Returns (x, pending)."""
        raise NotImplementedError
