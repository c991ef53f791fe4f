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

import gc
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import BatchIndex
from ..cache.storage import CacheStorage
from ..ops import lib as ops_lib
from ..parts.base import StepContext
from .model import Model


@dataclass
class StepEntry:
    """The next ``tokens`` of ``request`` and the places among them (0-based)
    whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def _bucket(n: int, buckets=DECODE_BUCKETS):
    for b in buckets:
        if n <= b:
            return b
    return None


def _pow2_at_least(n: int, floor: int = 8) -> int:
    w = floor
    while w < n:
        w *= 2
    return w


class DecodeGraph:
    """One captured decode step: ``bucket`` single-token entries, block tables of fixed
    widths.  A real batch of up to ``bucket`` requests is padded with entries that read
    and write only the cache's padding page and slot.

    CUDA streams and graphs stand where the reference uses a tracing compiler plus its
    own graph runner (mstar/engine/cuda_graph_runner.py:45, 807-836: decode batches
    padded to the next captured size); what is replayed here are this package's own
    kernel launches."""

    RING = 3

    def __init__(self, stepper: "Stepper", bucket: int, widths: list):
        # no reference back to the stepper: a stepper and its graphs must not form a cycle,
        # or they would be freed by the cyclic collector at a moment of its choosing, which
        # may be the middle of another graph's capture (freeing device memory there
        # invalidates that capture)
        self.manager, self.storage = stepper.manager, stepper.storage
        self.bucket = bucket
        self.widths = list(widths)
        mgr, storage = stepper.manager, stepper.storage
        self.pad_pages = [storage.pad_page(g) for g in range(len(mgr.groups))]
        self.extra = (("token_ids", bucket), ("want_rows", bucket), ("token_src", bucket))
        probe = mgr.fill_batch([], [], extra=self.extra, widths=self.widths, pad_entries=bucket,
                               pad_page=self.pad_pages, pad_slot=storage.pad_slot)
        self.offsets = probe.offsets
        self.size = probe.packed.size
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=stepper.device)
        self.pinned = [torch.empty(self.size, dtype=torch.int32, pin_memory=True)
                       for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        bound = max([w * g.page_size for w, g in zip(self.widths, mgr.groups)] or [1])

        def view(name: str) -> torch.Tensor:
            off, length = self.offsets[name]
            return self.dev[off:off + length]

        self.ctx = StepContext(
            num_tokens=bucket, num_entries=bucket, token_req=view("token_req"),
            positions=view("positions"), cache_pos=view("cache_pos"),
            qo_indptr=view("qo_indptr"), kv_len=view("kv_len"), slots=view("slots"),
            q_lens=[1] * bucket, kv_lens=[bound] * bucket,
            host_slots=[storage.pad_slot] * bucket, max_q_len=1, max_kv_len=bound,
            num_decode=bucket, token_source=(view("token_src"), stepper.device_tokens))
        self.tables = [view(f"table{g}").view(bucket, -1) for g in range(len(mgr.groups))]
        self.token_ids = view("token_ids")
        self.want_rows = view("want_rows")
        self._stage([], [], None)
        model = stepper.model
        side = torch.cuda.Stream(device=stepper.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                     # warm-up outside the capture
            model.forward(self.token_ids, self.ctx, storage, self.tables, self.want_rows)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(stepper.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops_lib.launch_count()
        # and no collection of other garbage while the capture is under way
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = model.forward(self.token_ids, self.ctx, storage, self.tables,
                                            self.want_rows)
        finally:
            if collecting:
                gc.enable()
        self.launches = ops_lib.launch_count() - before   # own kernels in one replay

    def _stage(self, requests: list, tokens: list, sources) -> int:
        """Fill the next pinned buffer for this batch and start its copy to the device.
        ``sources[i]``: index into the stepper's device tokens that request i's token is
        taken from, or -1 (``tokens[i]`` is it); None: all from ``tokens``."""
        turn = self.turn
        self.turn = (turn + 1) % self.RING
        if self.events[turn] is not None:
            self.events[turn].synchronize()               # its last copy has been read
        pinned = self.pinned[turn]
        n = len(requests)
        index = self.manager.fill_batch(
            requests, [1] * n, extra=self.extra, alloc=lambda size: pinned.numpy(),
            widths=self.widths, pad_entries=self.bucket - n, pad_page=self.pad_pages,
            pad_slot=self.storage.pad_slot)
        off, length = index.offsets["token_ids"]
        index.packed[off:off + n] = tokens
        index.packed[off + n:off + length] = 0
        off, length = index.offsets["want_rows"]
        index.packed[off:off + length] = np.arange(length, dtype=np.int32)
        off, length = index.offsets["token_src"]
        index.packed[off:off + length] = -1
        if sources is not None:
            index.packed[off:off + n] = sources
        self.dev.copy_(pinned, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[turn] = ev
        return self.size * 4

    def run(self, requests: list, tokens: list, sources=None) -> torch.Tensor:
        """``sources``: per request, the index into the stepper's device tokens (the
        sampler's output of the step before) that replaces ``tokens[i]`` without the host
        ever seeing the value, or -1."""
        self._stage(requests, tokens, sources)
        self.graph.replay()
        ops_lib.add_launches(self.launches)
        return self.logits[:len(requests)]


class Stepper:
    def __init__(self, model: Model, storage: CacheStorage, *, cuda_graphs: bool = True):
        self.model = model
        self.storage = storage
        self.manager = storage.manager
        # sequences are as long as the model's positions reach (the reference derives
        # max_seq_len from max_position_embeddings, mstar/model/orpheus/orpheus_model.py:
        # 88-95): a step that would pass them raises SequenceTooLong, nothing changed
        self.manager.set_max_positions(getattr(model, "max_positions", None))
        self.device = model.runtime.device
        self.steps = 0
        self.last_h2d_bytes = 0
        self.cuda_graphs = bool(cuda_graphs) and getattr(model, "graph_safe", False)
        self._graphs: dict = {}
        self.graph_replays = 0
        # tokens sampled by the step before, for steps launched before the host has read
        # them (see ``step``); captured graphs read this buffer
        self.device_tokens = torch.zeros(max(DECODE_BUCKETS), dtype=torch.int32, device=self.device)

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

    def step(self, entries: Sequence[StepEntry], pending: Optional[dict] = None,
             device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch; returns float32 logits [number of wanted places, vocab] on
        the device, in the order of ``entries`` and of each entry's ``want``.
        Raises ``CacheExhausted`` (nothing changed) if the pages do not suffice, and
        ``SequenceTooLong`` (nothing changed) if a request would pass the model's positions.
        The tensor returned by a step of single tokens may be a view of a captured graph's
        output buffer: the next such step of the same shape overwrites it, so a caller that
        keeps logits across steps copies them (``clone()``) first.

        ``pending``: entry index -> index into ``device_tokens`` (int32 on the device, the
        tokens the step before sampled).  Such an entry brings one token whose value the
        host does not know yet (its ``tokens`` hold any valid id); the step is launched
        without waiting for it."""
        vocab = self.model.vocab_size
        entries = list(entries)
        if not entries:
            return torch.empty((0, vocab), dtype=torch.float32, device=self.device)
        pending = pending or {}
        if pending:
            if device_tokens is None or device_tokens.dtype != torch.int32:
                raise ValueError("pending tokens need the int32 device tensor they come from")
            if device_tokens.numel() > self.device_tokens.numel():
                self.device_tokens = torch.zeros(device_tokens.numel(), dtype=torch.int32,
                                                 device=self.device)
                self._graphs.clear()                # they captured the old buffer
            for i, src in pending.items():
                if len(entries[i].tokens) != 1 or not 0 <= src < device_tokens.numel():
                    raise ValueError("a pending entry brings one token from the device tokens")
            self.device_tokens[:device_tokens.numel()].copy_(device_tokens, non_blocking=True)
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
        if self.cuda_graphs and all(len(e.tokens) == 1 for e in entries):
            logits = self._step_decode_graph(entries, pending)
            if logits is not None:
                return logits
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        ordered = [entries[i] for i in order]
        requests = [e.request for e in ordered]
        counts = [len(e.tokens) for e in ordered]
        starts = np.concatenate([[0], np.cumsum(counts)]).tolist()
        start_of = {order[j]: starts[j] for j in range(len(order))}
        want_rows = [start_of[i] + w for i, e in enumerate(entries) for w in e.want]
        total = starts[-1]

        self.manager.reserve(requests, counts)
        extra = [("token_ids", total), ("want_rows", len(want_rows))]
        if pending:
            extra.append(("token_src", total))
        index: BatchIndex = self.manager.fill_batch(requests, counts, extra=tuple(extra),
                                                    alloc=self._pinned)
        o, n = index.offsets["token_ids"]
        index.packed[o:o + n] = np.fromiter((t for e in ordered for t in e.tokens),
                                            dtype=np.int32, count=total)
        o, n = index.offsets["want_rows"]
        index.packed[o:o + n] = np.asarray(want_rows, dtype=np.int32)
        if pending:
            o, n = index.offsets["token_src"]
            index.packed[o:o + n] = -1
            for i, src in pending.items():
                index.packed[o + start_of[i]] = src

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
            max_q_len=max(counts), max_kv_len=int(index.kv_len.max()), num_decode=num_decode,
            token_source=(view("token_src"), self.device_tokens) if pending else None)
        tables = [view(f"table{g}").view(len(ordered), -1)
                  for g in range(len(self.manager.groups))]
        # per-request state is written in place by the mixers that keep some: it is put back
        # if the pass fails, so that state and lengths move together or not at all
        saved = self.storage.snapshot_state(index.slots.tolist())
        try:
            logits = self.model.forward(view("token_ids"), ctx, self.storage, tables,
                                        view("want_rows"))
        except BaseException:
            self.storage.restore_state(saved)
            raise
        for request, count in zip(requests, counts):
            self.manager.commit(request, count)
        self.steps += 1
        return logits


    def _step_decode_graph(self, entries: list, pending: Optional[dict] = None):
        """A batch of single tokens as the replay of a captured graph; None when the
        batch is larger than the largest captured shape."""
        bucket = _bucket(len(entries))
        if bucket is None:
            return None
        requests = [e.request for e in entries]
        self.manager.reserve(requests, [1] * len(entries))
        widths = tuple(_pow2_at_least(w) for w in self.manager.batch_widths(requests))
        key = (bucket, widths)
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._graphs[key] = DecodeGraph(self, bucket, list(widths))
        sources = None
        if pending:
            sources = [pending.get(i, -1) for i in range(len(entries))]
        saved = None
        if self.storage.has_state:
            saved = self.storage.snapshot_state([self.manager.slot(r) for r in requests])
        try:
            logits = graph.run(requests, [e.tokens[0] for e in entries], sources)
        except BaseException:
            self.storage.restore_state(saved)
            raise
        self.last_h2d_bytes = graph.size * 4
        for request in requests:
            self.manager.commit(request, 1)
        self.steps += 1
        self.graph_replays += 1
        wanted = [i for i, e in enumerate(entries) for _ in e.want]
        if wanted == list(range(len(entries))):
            return logits
        if not wanted:
            return logits[:0]
        return logits[torch.tensor(wanted, dtype=torch.long, device=self.device)]


def make_stepper(model: Model, *, page_size=16, num_pages=None,
                 max_tokens: Optional[int] = None, num_slots: int = 64,
                 cuda_graphs: bool = True) -> Stepper:
    """A stepper with a cache pool of ``num_pages`` pages per group, or enough pages
    for ``max_tokens`` cached tokens.  ``page_size`` and ``num_pages``: one number for
    every cache group, or a list with one per group."""
    if num_pages is None:
        if max_tokens is None:
            raise ValueError("give num_pages or max_tokens")
        sizes = [page_size] if isinstance(page_size, int) else list(page_size)
        num_pages = [-(-int(max_tokens) // p) for p in sizes]
        if isinstance(page_size, int):
            num_pages = num_pages[0]
    storage = CacheStorage(model.cache_needs, model.runtime.dtype, model.runtime.device,
                           page_size, num_pages, num_slots)
    return Stepper(model, storage, cuda_graphs=cuda_graphs)
