"""The step function: one batch of (request, its next tokens), run from the cache.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.
Only the tokens given are computed; everything earlier comes from the cache that
earlier steps left.  Logits are returned for the places the caller names.

The reference's engine step (mstar/engine/kv_cache_engine.py:660-711) takes whole
prompts or single tokens, never both and never a portion, and returns sampled
tokens; its planning already works on per-request new-token counts on top of the
cached length (mstar/engine/cache_manager.py:278-294), which is the index
structure used here for any cut.  As there, pages are reserved before the forward
pass and lengths advance after it, and a batch that does not fit raises with
nothing changed (the reference reports allocation_failed, kv_cache_engine.py:693-708).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import BatchIndex
from ..cache.storage import CacheStorage
from ..parts.base import StepContext
from .model import Model


@dataclass
class StepEntry:
    """The next ``tokens`` of ``request`` and the places among them (0-based)
    whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


class Stepper:
    def __init__(self, model: Model, storage: CacheStorage):
        self.model = model
        self.storage = storage
        self.manager = storage.manager
        self.device = model.runtime.device
        self.steps = 0
        self.last_h2d_bytes = 0

    # -- requests ---------------------------------------------------------
    def add_request(self, request: Hashable) -> int:
        """Give the request a state slot (zeroed); it holds no pages yet."""
        slot = self.manager.add_request(request)
        self.storage.reset_slot(slot)
        return slot

    def free_request(self, request: Hashable) -> None:
        """The request is finished: its pages and its slot return to the pools."""
        self.manager.free_request(request)

    def has_request(self, request: Hashable) -> bool:
        return self.manager.has(request)

    # -- one step ---------------------------------------------------------
    def _pinned(self, n: int) -> np.ndarray:
        self._staging = torch.empty(n, dtype=torch.int32, pin_memory=True)
        return self._staging.numpy()

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; returns float32 logits [number of wanted places, vocab] on
        the device, in the order of ``entries`` and of each entry's ``want``.
        Raises ``CacheExhausted`` (nothing changed) if the pages do not suffice."""
        vocab = self.model.vocab_size
        entries = list(entries)
        if not entries:
            return torch.empty((0, vocab), dtype=torch.float32, device=self.device)
        for e in entries:
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request!r} brings no tokens to this step")
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                raise ValueError(f"request {e.request!r} has a token id outside [0, {vocab})")
            for wpos in e.want:
                if not 0 <= wpos < len(e.tokens):
                    raise ValueError(f"request {e.request!r} wants place {wpos} of "
                                     f"{len(e.tokens)} tokens")
        # single tokens first: kernels specialised for one query per request take
        # tokens [0, num_decode), the others the rest
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        ordered = [entries[i] for i in order]
        requests = [e.request for e in ordered]
        counts = [len(e.tokens) for e in ordered]
        starts = np.concatenate([[0], np.cumsum(counts)]).tolist()
        start_of = {order[j]: starts[j] for j in range(len(order))}
        want_rows = [start_of[i] + w for i, e in enumerate(entries) for w in e.want]
        total = starts[-1]

        self.manager.reserve(requests, counts)
        index: BatchIndex = self.manager.fill_batch(
            requests, counts, extra=(("token_ids", total), ("want_rows", len(want_rows))),
            alloc=self._pinned)
        o, n = index.offsets["token_ids"]
        index.packed[o:o + n] = np.fromiter((t for e in ordered for t in e.tokens),
                                            dtype=np.int32, count=total)
        o, n = index.offsets["want_rows"]
        index.packed[o:o + n] = np.asarray(want_rows, dtype=np.int32)

        dev = torch.empty(index.packed.size, dtype=torch.int32, device=self.device)
        dev.copy_(self._staging[:index.packed.size], non_blocking=True)
        self.last_h2d_bytes = index.packed.size * 4

        def view(name: str) -> torch.Tensor:
            off, length = index.offsets[name]
            return dev[off:off + length]

        num_decode = sum(1 for c in counts if c == 1)
        ctx = StepContext(
            num_tokens=total, num_entries=len(ordered), token_req=view("token_req"),
            positions=view("positions"), cache_pos=view("cache_pos"),
            qo_indptr=view("qo_indptr"), kv_len=view("kv_len"), slots=view("slots"),
            q_lens=counts, kv_lens=index.kv_len.tolist(), host_slots=index.slots.tolist(),
            max_q_len=max(counts), max_kv_len=int(index.kv_len.max()), num_decode=num_decode)
        tables = [view(f"table{g}").view(len(ordered), -1)
                  for g in range(len(self.manager.groups))]
        logits = self.model.forward(view("token_ids"), ctx, self.storage, tables,
                                    view("want_rows"))
        for request, count in zip(requests, counts):
            self.manager.commit(request, count)
        self.steps += 1
        return logits


def make_stepper(model: Model, *, page_size: int = 16, num_pages: Optional[int] = None,
                 max_tokens: Optional[int] = None, num_slots: int = 64) -> Stepper:
    """A stepper with a cache pool of ``num_pages`` pages per group, or enough pages
    for ``max_tokens`` cached tokens."""
    if num_pages is None:
        if max_tokens is None:
            raise ValueError("give num_pages or max_tokens")
        num_pages = -(-int(max_tokens) // page_size)
    storage = CacheStorage(model.cache_needs, model.runtime.dtype, model.runtime.device,
                           page_size, int(num_pages), num_slots)
    return Stepper(model, storage)
