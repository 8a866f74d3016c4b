"""Device memory of the cache: one slab of pages per group, one state tensor per
layer execution that keeps state of fixed size.

Layer executions whose mixers need the same thing (number of key/value heads,
head size, window) form a group.  A group's slab is ``[executions, 2, pages,
kv_heads, page_size, head_dim]`` (index 1: 0 = keys, 1 = values), so the keys of
one page and head are ``page_size * head_dim`` contiguous elements: one bulk copy
per page and head for the attention kernels.  The reference allocates ``[2,
pages, page_size, kv_heads, head_dim]`` per layer (minivllm/worker/
kv_cache_alloc.py:65-85); grouping by need follows minivllm/worker/
gpu_model_runner.py:521-580.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import CacheView, KVPagesNeed, StateNeed


@dataclass
class CacheGroup:
    need: KVPagesNeed
    entries: list[int]              # schedule entries that own a slice of the slab
    # Keys and values of one size: ``slab`` is ``[executions, 2, pages, kv_heads, page_size,
    # head_dim]``.  Values of a size of their own: ``slab`` holds the keys ``[executions, pages,
    # kv_heads, page_size, head_dim]`` and ``value_slab`` the values likewise.
    slab: torch.Tensor
    value_slab: torch.Tensor | None = None


def _value_dim(need: KVPagesNeed) -> int:
    """Elements a position's values take per head: the keys' size unless told otherwise; 0 where the
    cached rows serve as both."""
    return need.head_dim if need.value_dim is None else need.value_dim


def split_needs(need) -> tuple[KVPagesNeed | None, list[StateNeed]]:
    """What a part asked for (one need, a tuple of them or None) as its pages and its states."""
    items = [] if need is None else list(need) if isinstance(need, (tuple, list)) else [need]
    pages = [item for item in items if isinstance(item, KVPagesNeed)]
    states = [item for item in items if isinstance(item, StateNeed)]
    if len(pages) > 1 or len(pages) + len(states) != len(items):
        raise ValueError(f"a part may ask for at most one set of pages and any number of states, got {items}")
    if len({state.name for state in states}) != len(states):
        raise ValueError(f"a part's states must have names of their own, got {[s.name for s in states]}")
    return (pages[0] if pages else None), states


class CacheStorage:
    def __init__(self, needs: list, cache_from: list[int | None],
                 page_size: int, num_pages: int, max_requests: int, dtype: torch.dtype,
                 device: torch.device | str, embedding_need=None) -> None:
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.groups: list[CacheGroup] = []
        # Every state tensor, under (schedule entry, name); the embedding's under ("embedding", name).
        self.states: dict[tuple, torch.Tensor] = {}
        group_of_key: dict[tuple, int] = {}
        members: dict[int, list[int]] = {}
        split = [split_needs(need) for need in needs]
        for index, (pages, _) in enumerate(split):
            if pages is not None:
                value_dim = pages.value_dim if pages.value_dim not in (None, pages.head_dim) else None
                key = (pages.num_kv_heads, pages.head_dim, pages.window, value_dim,
                       pages.keep_first if pages.window is not None else 0)
                group = group_of_key.setdefault(key, len(group_of_key))
                members.setdefault(group, []).append(index)
        page_views: dict[int, tuple[int, torch.Tensor, torch.Tensor]] = {}
        for key, group in sorted(group_of_key.items(), key=lambda item: item[1]):
            need = KVPagesNeed(*key)
            count = len(members[group])
            if need.value_dim == 0:
                # rows that serve as keys and as values: one slab, handed out under both names
                keys = torch.zeros((count, num_pages, need.num_kv_heads, page_size, need.head_dim),
                                   dtype=dtype, device=device)
                self.groups.append(CacheGroup(need, members[group], keys))
                for position, index in enumerate(members[group]):
                    page_views[index] = (group, keys[position], keys[position])
            elif need.value_dim is None:
                slab = torch.zeros((count, 2, num_pages, need.num_kv_heads, page_size, need.head_dim),
                                   dtype=dtype, device=device)
                self.groups.append(CacheGroup(need, members[group], slab))
                for position, index in enumerate(members[group]):
                    page_views[index] = (group, slab[position, 0], slab[position, 1])
            else:
                keys = torch.zeros((count, num_pages, need.num_kv_heads, page_size, need.head_dim),
                                   dtype=dtype, device=device)
                values = torch.zeros((count, num_pages, need.num_kv_heads, page_size, need.value_dim),
                                     dtype=dtype, device=device)
                self.groups.append(CacheGroup(need, members[group], keys, values))
                for position, index in enumerate(members[group]):
                    page_views[index] = (group, keys[position], values[position])

        def state_tensors(owner, wanted: list[StateNeed]) -> dict[str, torch.Tensor]:
            made = {}
            for need in wanted:
                # one spare row past the last slot: padded rows of fixed-shape batches land there
                made[need.name] = self.states[(owner, need.name)] = torch.zeros(
                    (max_requests + 1, *need.shape), dtype=need.dtype, device=device)
            return made

        owner_view: dict[int, CacheView] = {}
        for index, (pages, states) in enumerate(split):
            tensors = state_tensors(index, states)
            first = next(iter(tensors.values()), None)
            if pages is not None:
                group, keys, values = page_views[index]
                owner_view[index] = CacheView("pages", group, keys, values, state=first, states=tensors)
            elif tensors:
                owner_view[index] = CacheView("state", state=first, states=tensors)
        self.embedding_view: CacheView | None = None
        pages, states = split_needs(embedding_need)
        if pages is not None:
            raise ValueError("an embedding keeps state per request, not pages")
        if states:
            tensors = state_tensors("embedding", states)
            self.embedding_view = CacheView("state", state=next(iter(tensors.values())), states=tensors)
        self.views: list[CacheView] = []
        for index, need in enumerate(needs):
            source = cache_from[index]
            if source is not None:
                view = owner_view.get(source)
                if view is None:
                    raise ValueError(f"schedule entry {index} reads the cache of entry {source}, which has none")
                self.views.append(CacheView(view.kind, view.group, view.keys, view.values, view.state,
                                            writable=False, states=view.states))
            else:
                self.views.append(owner_view.get(index, CacheView("none")))

    @staticmethod
    def bytes_per_page(needs: list, page_size: int, dtype: torch.dtype) -> int:
        """Memory one page number costs over all executions that own a cache of pages (every
        group's pool has the same number of pages, so a page number exists once in each)."""
        element = torch.empty((), dtype=dtype).element_size()
        pages = [split_needs(need)[0] for need in needs]
        return sum(need.num_kv_heads * page_size * (need.head_dim + _value_dim(need)) * element
                   for need in pages if need is not None)

    @property
    def group_windows(self) -> list[int | None]:
        return [group.need.window for group in self.groups]

    @property
    def group_keep_first(self) -> list[int]:
        """Per group: the first positions of a sequence that stay readable whatever the window."""
        return [group.need.keep_first for group in self.groups]

    @property
    def has_state(self) -> bool:
        return bool(self.states)

    def zero_slots(self, slots: list[int]) -> None:
        """State of a request starts at zero: at admission and after preemption."""
        if slots and self.states:
            for state in self.states.values():
                index = torch.tensor(slots, dtype=torch.long, device=state.device)
                state.index_fill_(0, index, 0)

    def num_bytes(self) -> int:
        total = sum(slab.numel() * slab.element_size() for g in self.groups
                    for slab in (g.slab, g.value_slab) if slab is not None)
        return total + sum(s.numel() * s.element_size() for s in self.states.values())

    def bytes_per_token(self) -> int:
        """Cache bytes one position of one request occupies over all groups."""
        return sum(len(g.entries) * g.need.num_kv_heads * (g.need.head_dim + _value_dim(g.need))
                   * g.slab.element_size() for g in self.groups)
