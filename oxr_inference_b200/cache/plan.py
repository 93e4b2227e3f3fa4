"""What the model's schedule needs of the cache: which runs share a pool of pages, which keep fixed state."""

from __future__ import annotations

from dataclasses import dataclass

from oxr_inference_b200.parts.base import PagedKVNeed, StateNeed


@dataclass(frozen=True)
class GroupPlan:
    """Layers with the same need (KV heads, head size, window) share pages: one page id is valid in each of
    them, as in the reference one block id is valid in every layer (oxr_runtime/kv_cache.py:23). Layers with a
    different need get a pool and block tables of their own."""

    need: PagedKVNeed
    num_layers: int


@dataclass(frozen=True)
class EntryPlan:
    """Where one schedule entry keeps what it keeps."""

    group: int | None = None
    layer_in_group: int = 0
    store: bool = True
    state: int | None = None


@dataclass(frozen=True)
class CachePlan:
    groups: tuple[GroupPlan, ...]
    states: tuple[StateNeed, ...]
    entries: tuple[EntryPlan, ...]


def make_cache_plan(needs: list[PagedKVNeed | StateNeed | None], cache_of: list[int | None]) -> CachePlan:
    """``needs[i]``: what schedule entry i's mixer keeps; ``cache_of[i]``: the entry whose cache it reads instead."""
    groups: list[list] = []  # [need, layer count]
    states: list[StateNeed] = []
    entries: list[EntryPlan | None] = [None] * len(needs)
    for i, (need, src) in enumerate(zip(needs, cache_of)):
        if src is not None:
            continue
        if isinstance(need, PagedKVNeed):
            for g, (have, count) in enumerate(groups):
                if have == need:
                    entries[i] = EntryPlan(group=g, layer_in_group=count)
                    groups[g][1] += 1
                    break
            else:
                groups.append([need, 1])
                entries[i] = EntryPlan(group=len(groups) - 1, layer_in_group=0)
        elif isinstance(need, StateNeed):
            states.append(need)
            entries[i] = EntryPlan(state=len(states) - 1)
        elif need is None:
            entries[i] = EntryPlan()
        else:
            raise TypeError(f"schedule entry {i}: unknown cache need {need!r}")
    for i, src in enumerate(cache_of):
        if src is None:
            continue
        if not 0 <= src < len(needs) or cache_of[src] is not None:
            raise ValueError(f"schedule entry {i} reads the cache of entry {src}, which has none of its own")
        if src >= i:
            raise ValueError(f"schedule entry {i} reads the cache of a later entry ({src}); it would read stale keys")
        owner = entries[src]
        if owner.group is None:
            raise ValueError(f"schedule entry {i} reads the cache of entry {src}, which keeps no keys and values")
        if needs[i] != needs[src]:
            raise ValueError(f"schedule entry {i} needs {needs[i]} but reads the cache of entry {src} with {needs[src]}")
        entries[i] = EntryPlan(group=owner.group, layer_in_group=owner.layer_in_group, store=False)
    return CachePlan(tuple(GroupPlan(n, c) for n, c in groups), tuple(states), tuple(entries))
