"""Device memory of the cache: key/value pages and per-request state slots.

Run-order entries (caches) whose mixers have the same needs as to which keys
must stay (all of them, or a window) form a group; a group has one pool of page
ids and one block table per request, and each cache of the group has its own
tensor [pages, 2, kv_heads, page_size, head_dim] indexed by those ids.  The
reference keeps one tensor [layers, pages, 2, page_size, kv_heads, head_dim] per
model component (mstar/engine/kv_cache_engine.py:132-136); here a page keeps the
tokens of one head contiguous, so a page of one head is one 16-byte-aligned run
that bulk copies can move.

State slots hold per-request state of fixed size for mixers that ask for it; the
architecture served here asks for none, so the pool exists with zero bytes.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..parts.base import CacheNeed, LayerCache
from .manager import CacheManager, GroupConfig

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


def plan_groups(needs: Sequence[CacheNeed]):
    """Group caches by the window of their keys.  Returns (windows, group_of):
    ``windows[g]`` is None or W, ``group_of[cache]`` the group index or None."""
    windows: list = []
    group_of: list = []
    for need in needs:
        if need is None or need.kv is None:
            group_of.append(None)
            continue
        w = need.kv.window
        if w not in windows:
            windows.append(w)
        group_of.append(windows.index(w))
    return windows, group_of


def group_page_sizes(page_size, num_groups: int) -> list:
    """One page size per group from one int for all, or a sequence with one per group."""
    if isinstance(page_size, int):
        sizes = [page_size] * num_groups
    else:
        sizes = [int(p) for p in page_size]
        if len(sizes) != num_groups:
            raise ValueError(f"{num_groups} cache groups but {len(sizes)} page sizes")
    if any(p <= 0 for p in sizes):
        raise ValueError(f"page sizes must be positive, got {sizes}")
    return sizes


def bytes_per_page(needs: Sequence[CacheNeed], group_of, group: int, page_size: int,
                   dtype: torch.dtype) -> int:
    item = torch.empty((), dtype=dtype).element_size()
    total = 0
    for need, g in zip(needs, group_of):
        if g == group:
            total += 2 * need.kv.num_kv_heads * page_size * need.kv.head_dim * item
    return total


class CacheStorage:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], dtype: torch.dtype,
                 device: torch.device, page_size, num_pages, num_slots: int):
        """``page_size`` and ``num_pages``: one int for every group, or a list with one per
        group (a group of windowed layers may want smaller pages than one that keeps every
        key: it gives them back sooner)."""
        self.needs = list(needs)
        self.dtype = dtype
        self.device = device
        self.num_slots = int(num_slots)
        self.windows, self.group_of = plan_groups(self.needs)
        self.page_sizes = group_page_sizes(page_size, len(self.windows))
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.windows)
        if len(num_pages) != len(self.windows):
            raise ValueError(f"{len(self.windows)} cache groups but {len(num_pages)} page counts")
        self.group_configs = [GroupConfig(p, int(n), w)
                              for p, n, w in zip(self.page_sizes, num_pages, self.windows)]
        self.manager = CacheManager(self.group_configs, self.num_slots)
        self.kv: list = []
        self.state: list = []
        for need, g in zip(self.needs, self.group_of):
            if g is None:
                self.kv.append(None)
            else:
                # one page more than the manager hands out: padding entries of
                # fixed-shape (CUDA graph) batches write their keys there
                n = self.group_configs[g].num_pages + 1
                self.kv.append(torch.zeros(
                    (n, 2, need.kv.num_kv_heads, self.page_sizes[g], need.kv.head_dim),
                    dtype=dtype, device=device))
            if need is not None and need.state is not None:
                self.state.append(torch.zeros((self.num_slots + 1,) + tuple(need.state.shape),
                                              dtype=_STATE_DTYPES[need.state.dtype],
                                              device=device))
            else:
                self.state.append(None)

    def pad_page(self, group: int) -> int:
        """The page of ``group`` that padding entries may scribble on."""
        return self.group_configs[group].num_pages

    @property
    def pad_slot(self) -> int:
        return self.num_slots

    def state_bytes_per_request(self) -> int:
        return sum(0 if s is None else s[0].numel() * s.element_size() for s in self.state)

    @property
    def has_state(self) -> bool:
        return any(s is not None for s in self.state)

    def snapshot_state(self, slots) -> Optional[tuple]:
        """Copies of the state rows of ``slots`` (None when no mixer keeps state).  Mixers
        update their state in place during the forward pass; the step function takes this
        copy before the pass and puts it back if the pass fails, so that state, like the
        lengths, moves only with a step that completed (the reference advances its sequence
        state after the forward pass, mstar/engine/cache_manager.py:811-838)."""
        if not self.has_state:
            return None
        index = torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
        return index, [None if s is None else s.index_select(0, index) for s in self.state]

    def restore_state(self, snapshot) -> None:
        if snapshot is None:
            return
        index, rows = snapshot
        for s, saved in zip(self.state, rows):
            if s is not None:
                s.index_copy_(0, index, saved)

    def reset_slot(self, slot: int) -> None:
        """A request takes the slot: its state starts at zero."""
        for s in self.state:
            if s is not None:
                s[slot].zero_()

    def layer_cache(self, cache_id: int, block_tables: Sequence[torch.Tensor]) -> LayerCache:
        g = self.group_of[cache_id]
        return LayerCache(kv=self.kv[cache_id],
                          page_size=0 if g is None else self.page_sizes[g],
                          block_table=None if g is None else block_tables[g],
                          state=self.state[cache_id])
