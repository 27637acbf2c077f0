"""What a mixer asks of the cache manager for one request."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKV:
    """Keys and values for every cached position (or, with ``window``, for the last
    ``window`` positions only), stored in pages of ``page_size`` tokens."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """A per-request state of fixed size (``shape`` elements of ``dtype``), zeroed
    when the request is admitted."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
