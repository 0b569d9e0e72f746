"""Device memory of the cache: key and value pools per group, and state-slot tensors.

Pools of one group: ``k, v [layers_in_group, pages, kv_heads, page_size, head_dim]`` —
head-major inside a page, so the keys of one (page, kv head) are one contiguous tile.
A run step's ``LayerCache`` is the view its mixer works on.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .needs import PagedKVNeed, paged_need_of, state_needs_of


@dataclass
class LayerCache:
    """What one run step's mixer sees."""

    group: int | None = None  # cache group of the pools (index into the batch's group views)
    k: torch.Tensor | None = None  # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor | None = None
    page_size: int = 0
    writes: bool = True  # False: reads another run step's cache and writes nothing
    states: tuple = ()  # one tensor [max_requests, *shape] per StateNeed of the run step, in the order it named them

    @property
    def state(self) -> torch.Tensor | None:
        """The tensor of the run step's first (usually only) StateNeed."""
        return self.states[0] if self.states else None


def plan_groups(needs: list, run_order) -> tuple[list[PagedKVNeed], list[int | None]]:
    """Group run steps by equal paged needs.  Returns the groups' needs and, for each run step,
    its group (None for steps without pages); a step that reads another step's cache gets that
    step's group."""
    groups: list[PagedKVNeed] = []
    of_step: list[int | None] = []
    for i, answer in enumerate(needs):
        src = run_order[i].cache_of
        need = paged_need_of(answer)
        if src is not None:
            of_step.append(of_step[src])
        elif need is not None:
            if need not in groups:
                groups.append(need)
            of_step.append(groups.index(need))
        else:
            of_step.append(None)
    return groups, of_step


class CachePools:
    def __init__(self, needs: list, run_order, pages_per_group: list[int], page_size: int, max_requests: int,
                 dtype: torch.dtype, device: torch.device | str) -> None:
        self.page_size = page_size
        self.group_needs, self.group_of_step = plan_groups(needs, run_order)
        if len(pages_per_group) != len(self.group_needs):
            raise ValueError(f"{len(self.group_needs)} cache groups, {len(pages_per_group)} page counts")
        owners: list[list[int]] = [[] for _ in self.group_needs]
        for i, answer in enumerate(needs):
            if paged_need_of(answer) is not None and run_order[i].cache_of is None:
                owners[self.group_of_step[i]].append(i)
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        # one page more than the manager hands out: padding rows of a replayed graph live there
        self.scratch_pages = list(pages_per_group)
        for need, pages, own in zip(self.group_needs, pages_per_group, owners):
            shape = (len(own), pages + 1, need.num_kv_heads, page_size, need.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=device))
        self.layer_caches: list[LayerCache] = []
        for i, answer in enumerate(needs):
            src = run_order[i].cache_of
            if src is not None:
                base = self.layer_caches[src]
                self.layer_caches.append(LayerCache(base.group, base.k, base.v, page_size, writes=False, states=base.states))
                continue
            states = tuple(torch.zeros((max_requests, *need.shape), dtype=need.dtype, device=device) for need in state_needs_of(answer))
            if paged_need_of(answer) is not None:  # pages, and state slots beside them if the step asked for both
                g = self.group_of_step[i]
                j = owners[g].index(i)
                self.layer_caches.append(LayerCache(g, self.k[g][j], self.v[g][j], page_size, states=states))
            else:
                self.layer_caches.append(LayerCache(states=states))

    @property
    def has_state(self) -> bool:
        return any(c.states for c in self.layer_caches)

    def reset_state(self, slot: int) -> None:
        """Zero a slot's state in every layer: a request starts (or starts over) from nothing."""
        seen = set()
        for c in self.layer_caches:
            for state in c.states:
                if state.data_ptr() not in seen:
                    seen.add(state.data_ptr())
                    state[slot].zero_()

    @staticmethod
    def bytes_per_page(needs: list, run_order, page_size: int, dtype: torch.dtype) -> list[int]:
        """Bytes one page costs in each group (keys and values, all the group's layers)."""
        group_needs, group_of_step = plan_groups(needs, run_order)
        out = [0] * len(group_needs)
        for i, answer in enumerate(needs):
            need = paged_need_of(answer)
            if need is not None and run_order[i].cache_of is None:
                out[group_of_step[i]] += 2 * need.num_kv_heads * page_size * need.head_dim * dtype.itemsize
        return out
