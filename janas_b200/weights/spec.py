"""What a part says about each tensor it needs."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

# kinds of tensors; they decide the resident dtype and the random distribution
MATRIX = "matrix"          # a linear layer's weight [out_features, in_features]
EMBEDDING = "embedding"    # the token table [vocab, hidden]
NORM = "norm"              # a norm's per-channel weight
INT_TABLE = "int_table"    # a table of whole numbers (kept as int32)
PARAM = "param"            # a small vector or scalar of constants (always kept as float32)


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    kind: str = MATRIX
    optional: bool = False   # absent is allowed (a tied head)
    mean: float = 0.0        # random weights of a PARAM: N(mean, std)
    std: float = 0.02
