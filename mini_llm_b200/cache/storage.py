"""Device memory of the caches, and the view of it each run entry gets.

Per paged group: keys and values as ``[entries, n_pages, page_size, kv_heads,
head_size]`` each (one page id covers every entry of the group, and every
entry's pages are one contiguous array), plus the device copy of the block
tables of the step's items, ``[max_items, max_blocks]`` int32, refilled before
each step.  Per fixed-state group: ``[entries, max_requests, *shape]``, zeroed
for a slot when a request opens it.

The reference allocates K and V per sequence and per layer
(engine/src/gpt2_gpu.cu:147-159) and passes the pointers in a control block
(engine/src/gpt2_gpu_batch.cu:18-24); here the pools are allocated once.
"""

from __future__ import annotations

import torch

from ..parts.spec import FixedState, PagedKV

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class LayerCache:
    """What one run entry's mixer may touch."""

    kind = "none"
    writes = False
    group = None


class PagedLayerCache(LayerCache):
    kind = "paged"

    def __init__(self, group, k_pages, v_pages, block_table, page_size, writes):
        self.group = group
        self.k_pages, self.v_pages = k_pages, v_pages      # [n_pages, page_size, kv_heads, head_size]
        self.block_table = block_table                     # [max_items, max_blocks] int32, rows = the step's items
        self.page_size = page_size
        self.writes = writes


class StateLayerCache(LayerCache):
    kind = "state"

    def __init__(self, group, state, writes):
        self.group = group
        self.state = state                                 # [max_requests, *shape], indexed by slot
        self.writes = writes


class CacheStorage:
    def __init__(self, manager, order, dtype: torch.dtype, device, max_items: int, poison: float | None = None):
        """``poison``: a debugging value.  Every page slot holds it until a token is stored
        there, and a page holds it again from the moment it is given back: a kernel that
        reads a slot past a request's length, or through a stale block-table row, then
        reads ``poison`` instead of another request's plausible keys."""
        self.manager = manager
        self.device = device
        self.max_items = int(max_items)
        self.poison = poison
        self.spare_page = True                # every pool has a page past its last (index n_pages)
        self.keys, self.values, self.states, self.block_tables = {}, {}, {}, {}
        for group in manager.groups:
            n_entries = len(group.entries)
            if isinstance(group.need, PagedKV):
                # one page beyond the pool's last: no request ever owns it; steps that are filled up
                # to a round shape let their filler tokens store there
                shape = (n_entries, group.pool.n_pages + 1, manager.page_size, group.need.n_kv_heads,
                         group.need.head_size)
                fill = 0.0 if poison is None else poison
                self.keys[group.index] = torch.full(shape, fill, dtype=dtype, device=device)
                self.values[group.index] = torch.full(shape, fill, dtype=dtype, device=device)
                self.block_tables[group.index] = torch.zeros((self.max_items, group.max_blocks), dtype=torch.int32,
                                                             device=device)
            elif isinstance(group.need, FixedState):
                shape = (n_entries, manager.max_requests, *group.need.shape)
                self.states[group.index] = torch.zeros(shape, dtype=_STATE_DTYPES[group.need.dtype], device=device)
        self.views = []
        for index, entry in enumerate(order):
            owner = index if entry.cache_of is None else entry.cache_of
            if owner not in manager.entry_group:
                self.views.append(LayerCache())
                continue
            g, position = manager.entry_group[owner]
            group = manager.groups[g]
            writes = entry.cache_of is None
            if group.paged:
                self.views.append(PagedLayerCache(g, self.keys[g][position], self.values[g][position],
                                                  self.block_tables[g], manager.page_size, writes))
            else:
                self.views.append(StateLayerCache(g, self.states[g][position], writes))

        if poison is not None:
            manager.on_free = self.poison_pages

    def poison_pages(self, group_index: int, pages) -> None:
        """Overwrite pages that went back to their pool (debugging engines only)."""
        index = torch.tensor(list(pages), dtype=torch.int64, device=self.device)
        for store in (self.keys, self.values):
            store[group_index].index_fill_(1, index, self.poison)

    def read_tokens(self, view_index: int, slot: int, first: int, count: int):
        """Keys and values of tokens ``first .. first + count - 1`` of the request in ``slot``
        as run entry ``view_index`` holds them: two tensors [count, kv_heads, head_size],
        gathered through the block table (the reference's test hook copies a layer's rows
        out of its contiguous cache, engine/src/gpt2_gpu.cu:185-195)."""
        view = self.views[view_index]
        if view.kind != "paged":
            raise ValueError(f"run entry {view_index} keeps no paged keys and values")
        page_size = self.manager.page_size
        row = self.manager.block_table_row(view.group, slot)
        positions = torch.arange(first, first + count, dtype=torch.int64)
        pages = torch.from_numpy(row.astype("int64"))[positions // page_size]
        if count and int(pages.min()) < 0:
            raise ValueError(f"slot {slot} holds no page for some of tokens {first}..{first + count - 1}")
        pages, within = pages.to(self.device), (positions % page_size).to(self.device)
        return view.k_pages[pages, within].clone(), view.v_pages[pages, within].clone()

    def reset_slot(self, slot: int) -> None:
        """Fixed-size state starts at zero for a new request."""
        for state in self.states.values():
            state[:, slot].zero_()

    def bytes(self) -> int:
        total = 0
        for store in (self.keys, self.values, self.states):
            total += sum(t.numel() * t.element_size() for t in store.values())
        return total
