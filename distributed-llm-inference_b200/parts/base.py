"""Interfaces of the parts a model is put together from, and their registry.

A part is built from a ``PartSpec`` (its sizes and constants) and a
``BuildEnv`` (dtype, device).  It declares the tensors it reads from the
checkpoint by full name, takes them in ``load``, and runs on the tokens of a
step.  No part knows which model it is in.

Interfaces by category (what a new part of that category must provide):

``norm``          ``add_norm(h, delta, rows=None) -> y``: h is the float32 residual stream
                  [n, H]; delta (activation dtype, or None) is added to h first, and the sum is
                  written back to h when ``rows`` is None; y (activation dtype) is the normed sum of
                  the rows asked for.
``position``      ``rotate_and_store(qkv, batch, cache, num_heads, num_kv_heads, write_kv) -> q``:
                  encodes position into the q and k heads of qkv [n, cols], writes
                  k, v into the cache's pages at ``batch.group(cache.group).slots`` and returns the
                  tensor whose leading columns are the encoded queries.
``mixer``         ``cache_need() -> PagedKVNeed | StateNeed | a sequence of them | None`` and
                  ``forward(x, batch, cache) -> [n, H]``; x is the normed input (activation dtype).
                  ``cache`` is the ``LayerCache`` of its run step: pages (``k, v``) for a PagedKVNeed,
                  ``state`` / ``states`` for StateNeeds, both for a mixer that asks for both (``writes``
                  is False when the step reads another step's cache).
``feed_forward``  ``forward(x) -> [n, H]``.
``arrangement``   built from a ``LayerSpec``; ``forward(stream, batch, cache)`` wires norms, mixer
                  and feed-forward around the residual ``stream`` (h plus a pending delta);
                  ``cache_need()`` says what its run step needs of the cache manager (usually its
                  mixer's answer; an arrangement with several mixers side by side returns all their
                  needs, and hands each mixer the same ``LayerCache``).
``embedding``     ``forward(token_ids) -> h`` float32 [n, H].
``head``          ``forward(y) -> logits`` float32 [k, V].

Optional, for the fusion of a part's last matrix product with the residual addition and the
norm behind it (a decode step's few tokens; see ``normed_input``).  A part that has none of
these is served with plain tensors:

* a mixer or feed-forward with an attribute ``defer_output`` (default False) may, when its owner
  set it, return a ``PendingProduct`` (the delta x W^T, not yet computed) instead of a tensor;
* a norm with ``add_product_norm(h, product) -> ScaledRows | None`` computes that product, adds it
  to h and leaves the division by the row's RMS to the reader of its output (None: it declines);
* a mixer, feed-forward or head with ``takes_scaled_rows`` true accepts such rows as its input
  (it hands them to ``kernels.gemm.project`` or a decode product of ``kernels.ops``);
* an arrangement with ``first_consumer() -> (norm, part)`` and ``defer_last_product(flag)`` lets
  the model extend this across layer borders.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorDecl


@dataclass(frozen=True)
class BuildEnv:
    dtype: torch.dtype  # activation and matrix dtype: torch.bfloat16 or torch.float32
    device: torch.device


class Part:
    """Base of every part: declares tensors by full name and receives them.

    ``graph_capturable``: whether the part's work on a step can be recorded in a CUDA graph (only
    launches on the current stream, no host synchronisation, no shapes that depend on the data).
    The engine replays decode steps from graphs only if every part of the model says so; a part
    that does not set it is taken to be not capturable, and the model then runs step by step."""

    graph_capturable = False

    def __init__(self, spec: PartSpec, env: BuildEnv) -> None:
        self.spec = spec
        self.env = env

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        """What, besides the number of sequences and the width of the block tables, changes this part's
        launches in a step where every sequence brings one token (for attention: into how many runs the
        keys are cut).  The step function records one graph per distinct answer and hands the answer back
        in ``batch.launch_keys[id(part)]`` when it runs the part for that graph, so that the part launches
        what it said it would.  None (the default): nothing does.  ``max_kv_len`` is the longest context
        the graph's tables can hold."""
        return None

    def declare(self) -> dict[str, TensorDecl]:
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        pass

    def children(self) -> list["Part"]:
        return []


class PendingProduct:
    """The delta x W^T of a residual stream, not yet computed: the norm that adds it may compute it
    in the same kernel.  ``materialize()`` computes it the plain way."""

    __slots__ = ("x", "weight")

    def __init__(self, x: torch.Tensor, weight: torch.Tensor) -> None:
        self.x, self.weight = x, weight

    def materialize(self) -> torch.Tensor:
        from ..kernels.gemm import project

        return project(self.x, self.weight)


class ResidualStream:
    """The float32 residual h [n, H] and a delta (activation dtype) not yet added to it.
    Keeping the delta pending lets the next norm do the addition in the same kernel.  ``pending``
    reads as a tensor (or None); ``take_pending()`` hands out a PendingProduct as it is."""

    def __init__(self, h: torch.Tensor, pending=None) -> None:
        self.h = h
        self._pending = pending

    @property
    def pending(self):
        if isinstance(self._pending, PendingProduct):
            self._pending = self._pending.materialize()
        return self._pending

    @pending.setter
    def pending(self, value) -> None:
        self._pending = value

    def take_pending(self):
        return self._pending


def can_fuse(norm, consumer) -> bool:
    """Whether ``norm`` can compute a PendingProduct itself and ``consumer`` reads what it then returns."""
    return hasattr(norm, "add_product_norm") and bool(getattr(consumer, "takes_scaled_rows", False))


def normed_input(norm, h: torch.Tensor, delta, consumer, rows: torch.Tensor | None = None):
    """norm(h + delta) as ``consumer`` will read it.  A delta that is still a PendingProduct goes,
    product and all, to a norm that can compute it (if the consumer reads ScaledRows and every row
    is wanted); otherwise it is computed first and the norm gets a tensor."""
    if isinstance(delta, PendingProduct):
        if rows is None and can_fuse(norm, consumer):
            y = norm.add_product_norm(h, delta)
            if y is not None:  # None: the norm declines (sizes its kernel does not take)
                return y
        delta = delta.materialize()
    return norm.add_norm(h, delta) if rows is None else norm.add_norm(h, delta, rows=rows)


_REGISTRY: dict[tuple[str, str], Callable[..., Any]] = {}

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head")


def register_part(category: str, kind: str):
    """Class decorator: ``@register_part("mixer", "my_mixer")``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r} (known: {CATEGORIES})")

    def deco(cls):
        _REGISTRY[(category, kind)] = cls
        return cls

    return deco


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.pop((category, kind), None)


def build_part(category: str, spec, env: BuildEnv):
    try:
        cls = _REGISTRY[(category, spec.kind if category != "arrangement" else spec.arrangement)]
    except KeyError:
        kind = spec.kind if category != "arrangement" else spec.arrangement
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise ValueError(f"no {category} part of kind {kind!r} is registered (known: {known})") from None
    return cls(spec, env)
