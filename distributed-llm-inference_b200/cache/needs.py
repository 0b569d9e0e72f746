"""What a mixer asks of the cache manager, in the manager's own terms."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token (or of the last ``window`` tokens) in pages.

    Run steps whose needs are equal share one group: one page id space and one
    block table per request.  A group with a window gives pages back once every
    position in them is older than the window.
    """

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one slot of this shape for each live request."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32
