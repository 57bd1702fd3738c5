"""What a part says about each tensor it needs."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

# kinds of tensors; they decide the resident dtype and the random distribution
MATRIX = "matrix"          # a linear layer's weight [out_features, in_features]
EMBEDDING = "embedding"    # the token table [vocab, hidden]
NORM = "norm"              # a norm's per-channel weight
INT_TABLE = "int_table"    # a table of whole numbers (kept as int32)


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    kind: str = MATRIX
    optional: bool = False   # absent is allowed (a tied head)
