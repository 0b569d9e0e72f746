"""Architecture-neutral description of a model: which parts, in which order.

A registered architecture turns its typed configuration into a ``ModelSpec``.
Everything below the registry (weights, cache manager, step function) works
from the spec alone, so no part needs to know which model it is in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind, its sizes and constants, and the prefix
    of its tensors' names in the checkpoint."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (how the parts are wired, e.g. ``prenorm``)
    and the parts by role (``mixer_norm``, ``mixer``, ``ffn_norm``, ``ffn``)."""

    arrangement: str
    parts: Mapping[str, PartSpec]


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` and may appear in several entries
    (shared weights).  Each entry owns a cache of its own unless ``cache_of``
    names an earlier entry whose cache it reads instead of writing one.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    run_order: tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec

    def __post_init__(self) -> None:
        for i, step in enumerate(self.run_order):
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"run_order[{i}] names layer {step.layer}, model has {len(self.layers)}")
            if step.cache_of is not None:
                if not 0 <= step.cache_of < i:
                    raise ValueError(f"run_order[{i}].cache_of must name an earlier entry")
                if self.run_order[step.cache_of].cache_of is not None:
                    raise ValueError(f"run_order[{i}].cache_of names an entry that owns no cache")
