"""What a mixer asks of the cache. Entries with equal requests share one group (one storage)."""
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVRequest:
    """Keys and values per token: [n_kv_heads, head_dim] each. ``window``: only the last
    ``window`` tokens are ever read, older pages may be given back; None: all tokens are kept."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int]
    dtype: torch.dtype


@dataclass(frozen=True)
class StateRequest:
    """A state of fixed shape per sequence, zero when the sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype
