"""Device memory of the cache: page pools per cache, state slots per cache."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from tokensprint_b200.cache.manager import GroupSpec
from tokensprint_b200.parts.base import CacheNeed, LayerCache


def groups_of(needs: Sequence[CacheNeed]) -> tuple[list[GroupSpec], list[int]]:
    """Sorts caches into groups by paging need.  Returns the groups and, for every cache,
    the index of its group (-1 for a cache without pages)."""
    keys: list[tuple[str, int]] = []
    index: list[int] = []
    for need in needs:
        if need.kind == "none":
            index.append(-1)
            continue
        if need.group_key not in keys:
            keys.append(need.group_key)
        index.append(keys.index(need.group_key))
    return [GroupSpec(kind, window) for kind, window in keys], index


def page_bytes(needs: Sequence[CacheNeed], group_index: Sequence[int], group: int, page_size: int, itemsize: int) -> int:
    """Bytes one page of `group` costs over all caches of the group (keys and values)."""
    return sum(page_size * n.token_elements * itemsize for n, g in zip(needs, group_index) if g == group)


@dataclass
class CacheTensors:
    """Per cache: the pools [pages, page_size, *k_row] and [pages, page_size, *v_row] (the second
    may be absent or of another row shape) and the state [slots, ...]."""

    k: list[Optional[torch.Tensor]]
    v: list[Optional[torch.Tensor]]
    state: list[Optional[torch.Tensor]]
    group_index: list[int]

    @classmethod
    def allocate(
        cls,
        needs: Sequence[CacheNeed],
        group_index: Sequence[int],
        pages_per_group: Sequence[int],
        page_size: int,
        num_slots: int,
        device: torch.device,
        dtype: torch.dtype,
    ) -> "CacheTensors":
        k, v, state = [], [], []
        for need, g in zip(needs, group_index):
            if g >= 0:
                k.append(torch.zeros((pages_per_group[g], page_size, *need.k_row), device=device, dtype=dtype))
                v.append(None if need.v_row is None else
                         torch.zeros((pages_per_group[g], page_size, *need.v_row), device=device, dtype=dtype))
            else:
                k.append(None)
                v.append(None)
            if need.state_shape is not None:
                state.append(torch.zeros((num_slots, *need.state_shape), device=device, dtype=need.state_dtype))
            else:
                state.append(None)
        return cls(k, v, state, list(group_index))

    def layer_cache(self, cache: int, writes: bool) -> LayerCache:
        return LayerCache(
            group=self.group_index[cache],
            k_pages=self.k[cache],
            v_pages=self.v[cache],
            state=self.state[cache],
            writes=writes,
        )

    def zero_slot(self, slot: int) -> None:
        for s in self.state:
            if s is not None:
                s[slot].zero_()

    def poison_pages(self, group: int, pages: Sequence[int]) -> None:
        """Debug aid: NaN into pages that were given back, so a stale read shows."""
        if not pages:
            return
        idx = None
        for c, g in enumerate(self.group_index):
            if g == group and self.k[c] is not None:
                if idx is None:
                    idx = torch.tensor(list(pages), device=self.k[c].device, dtype=torch.long)
                self.k[c][idx] = float("nan")
                if self.v[c] is not None:
                    self.v[c][idx] = float("nan")
