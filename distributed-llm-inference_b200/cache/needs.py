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


def needs_of(answer) -> tuple:
    """A run step's answer to ``cache_need()`` as a tuple of needs: nothing, one need, or several
    (a layer that keeps pages and a fixed-size state side by side).  At most one of them may be paged:
    a request has one block table per group, and a run step belongs to one group."""
    if answer is None:
        return ()
    needs = tuple(answer) if isinstance(answer, (tuple, list)) else (answer,)
    for need in needs:
        if not isinstance(need, (PagedKVNeed, StateNeed)):
            raise TypeError(f"a cache need is a PagedKVNeed or a StateNeed, not {type(need).__name__}")
    if sum(isinstance(n, PagedKVNeed) for n in needs) > 1:
        raise ValueError("a run step may ask for pages once (its other needs are StateNeeds)")
    return needs


def paged_need_of(answer) -> PagedKVNeed | None:
    return next((n for n in needs_of(answer) if isinstance(n, PagedKVNeed)), None)


def state_needs_of(answer) -> tuple[StateNeed, ...]:
    return tuple(n for n in needs_of(answer) if isinstance(n, StateNeed))
