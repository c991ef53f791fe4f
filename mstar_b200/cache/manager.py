"""Python face of the host-side cache manager (csrc/host/cache_manager.cpp).

The manager owns no device memory: it decides which page of which group a
request's tokens live in, which state slot the request has, and builds the
index arrays a step needs.  ``mstar_b200.cache.storage`` owns the tensors.

Life of a request: ``add_request`` (takes a state slot) -> per step
``reserve`` (pages for the step's new tokens, all-or-nothing for the batch)
-> ``fill_batch`` -> forward pass -> ``commit`` (length advances, pages that a
window has passed return to the pool) -> ... -> ``free_request`` (everything
returns).  The reference has the same order of plan-time growth and
post-forward commit (mstar/engine/cache_manager.py:278-285, 811-838).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Hashable, Optional, Sequence

import numpy as np

from ..ops.build import build_library

_OK, _NO_SLOT, _DUPLICATE, _UNKNOWN, _NO_PAGES, _BAD_ARG, _TOO_LONG = 0, -1, -2, -3, -4, -5, -6


class CacheExhausted(RuntimeError):
    """Not enough free pages for a batch; nothing was changed.

    ``short_by[g]`` is the number of pages group ``g`` lacks.  The reference's
    counterpart is AllocationFailedError (mstar/engine/kv_store.py:133-154)."""

    def __init__(self, short_by: Sequence[int]):
        self.short_by = list(short_by)
        super().__init__(f"cache pages exhausted: short by {self.short_by} pages per group")


class SequenceTooLong(ValueError):
    """A batch would give a token a position beyond what the model was built for
    (``max_position_embeddings``); nothing was changed."""


class NoFreeSlot(RuntimeError):
    """Every per-request state slot is taken."""


@dataclass(frozen=True)
class GroupConfig:
    """One pool of pages shared by the layers (caches) of a group.

    window None: all keys are kept until the request ends.  window W: a token
    sees the last W keys, and pages wholly older than that are released."""

    page_size: int
    num_pages: int
    window: Optional[int] = None


@dataclass
class BatchIndex:
    """Index arrays of one step, views into one packed int32 buffer."""

    packed: np.ndarray
    num_tokens: int
    num_entries: int
    token_req: np.ndarray
    positions: np.ndarray
    cache_pos: np.ndarray
    qo_indptr: np.ndarray
    kv_len: np.ndarray
    slots: np.ndarray
    tables: list            # per group: [entries, width]
    offsets: dict           # name -> (offset, length) in elements of `packed`


_lib = None


def _host_lib():
    global _lib
    if _lib is not None:
        return _lib
    lib = ctypes.CDLL(str(build_library("host")))
    i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
    pi32, pi64 = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int64)
    lib.cm_create.restype = vp
    lib.cm_create.argtypes = [i32, pi32, pi32, pi32, i32]
    lib.cm_destroy.restype = None
    lib.cm_destroy.argtypes = [vp]
    lib.cm_add_request.restype = i32
    lib.cm_add_request.argtypes = [vp, i64]
    lib.cm_free_request.restype = i32
    lib.cm_free_request.argtypes = [vp, i64]
    lib.cm_pages_needed.restype = i32
    lib.cm_pages_needed.argtypes = [vp, i32, pi64, pi32, pi64]
    lib.cm_reserve.restype = i32
    lib.cm_reserve.argtypes = [vp, i32, pi64, pi32, pi64]
    lib.cm_commit.restype = i32
    lib.cm_commit.argtypes = [vp, i64, i32]
    lib.cm_commit_positions.restype = i32
    lib.cm_commit_positions.argtypes = [vp, i64, i32, i64]
    lib.cm_position.restype = i64
    lib.cm_position.argtypes = [vp, i64]
    lib.cm_set_position.restype = i32
    lib.cm_set_position.argtypes = [vp, i64, i64]
    lib.cm_set_max_positions.restype = i32
    lib.cm_set_max_positions.argtypes = [vp, i64]
    lib.cm_len.restype = i64
    lib.cm_len.argtypes = [vp, i64]
    lib.cm_slot.restype = i32
    lib.cm_slot.argtypes = [vp, i64]
    lib.cm_free_pages.restype = i64
    lib.cm_free_pages.argtypes = [vp, i32]
    lib.cm_free_slots.restype = i32
    lib.cm_free_slots.argtypes = [vp]
    lib.cm_num_requests.restype = i32
    lib.cm_num_requests.argtypes = [vp]
    lib.cm_block_table.restype = i64
    lib.cm_block_table.argtypes = [vp, i64, i32, pi32, i64]
    lib.cm_batch_widths.restype = i32
    lib.cm_batch_widths.argtypes = [vp, i32, pi64, pi32]
    lib.cm_fill_batch.restype = i32
    lib.cm_fill_batch.argtypes = [vp, i32, pi64, pi32, pi32, pi32, pi32, pi32, pi32, pi32,
                                  ctypes.POINTER(pi32), pi32]
    lib.cm_check.restype = i32
    lib.cm_check.argtypes = [vp]
    _lib = lib
    return lib


def _i32(values) -> "ctypes.Array":
    return (ctypes.c_int * len(values))(*values)


def _i64(values) -> "ctypes.Array":
    return (ctypes.c_int64 * len(values))(*values)


def _round4(n: int) -> int:
    return (n + 3) & ~3


class CacheManager:
    def __init__(self, groups: Sequence[GroupConfig], num_slots: int):
        self.groups = list(groups)
        self.num_slots = int(num_slots)
        for g in self.groups:
            if g.page_size <= 0 or g.num_pages < 0 or (g.window is not None and g.window <= 0):
                raise ValueError(f"bad cache group {g}")
        self._lib = _host_lib()
        self._h = self._lib.cm_create(
            len(self.groups), _i32([g.page_size for g in self.groups]),
            _i32([g.num_pages for g in self.groups]),
            _i32([g.window or 0 for g in self.groups]), self.num_slots)
        if not self._h:
            raise ValueError("cache manager rejected its configuration")
        self._ids: dict[Hashable, int] = {}
        self._next = 1
        self.max_positions: Optional[int] = None

    def set_max_positions(self, max_positions: Optional[int]) -> None:
        """No token may get a position id >= ``max_positions`` (None: no limit): ``reserve``
        refuses such a batch with ``SequenceTooLong``.  The reference sizes its sequences by
        the model's max_position_embeddings (mstar/model/orpheus/orpheus_model.py:88-95)."""
        rc = self._lib.cm_set_max_positions(self._h, int(max_positions or 0))
        if rc != _OK:
            raise ValueError(f"bad position limit {max_positions}")
        self.max_positions = int(max_positions) if max_positions else None

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.cm_destroy(h)

    # -- requests ---------------------------------------------------------
    def _rid(self, request: Hashable) -> int:
        try:
            return self._ids[request]
        except KeyError:
            raise KeyError(f"request {request!r} is not in the cache manager") from None

    def has(self, request: Hashable) -> bool:
        return request in self._ids

    def add_request(self, request: Hashable) -> int:
        """Register a request and return its state slot."""
        if request in self._ids:
            raise ValueError(f"request {request!r} is already in the cache manager")
        rid = self._next
        slot = self._lib.cm_add_request(self._h, rid)
        if slot == _NO_SLOT:
            raise NoFreeSlot(f"all {self.num_slots} request slots are in use")
        if slot < 0:
            raise RuntimeError(f"cm_add_request failed with {slot}")
        self._next += 1
        self._ids[request] = rid
        return slot

    def free_request(self, request: Hashable) -> None:
        rid = self._rid(request)
        rc = self._lib.cm_free_request(self._h, rid)
        if rc != _OK:
            raise RuntimeError(f"cm_free_request failed with {rc}")
        del self._ids[request]

    def requests(self) -> list:
        return list(self._ids)

    # -- pages ------------------------------------------------------------
    def pages_needed(self, requests: Sequence[Hashable], n_new: Sequence[int]) -> list[int]:
        """New pages per group that ``reserve`` would take for this batch."""
        rids = _i64([self._rid(r) for r in requests])
        out = _i64([0] * max(1, len(self.groups)))
        rc = self._lib.cm_pages_needed(self._h, len(requests), rids, _i32(list(n_new)), out)
        if rc != _OK:
            raise RuntimeError(f"cm_pages_needed failed with {rc}")
        return [int(out[i]) for i in range(len(self.groups))]

    def reserve(self, requests: Sequence[Hashable], n_new: Sequence[int]) -> None:
        """Pages for ``n_new[i]`` more tokens of each request, in every group, or
        ``CacheExhausted`` with nothing changed."""
        rids = _i64([self._rid(r) for r in requests])
        short = _i64([0] * max(1, len(self.groups)))
        rc = self._lib.cm_reserve(self._h, len(requests), rids, _i32(list(n_new)), short)
        if rc == _NO_PAGES:
            raise CacheExhausted([int(short[i]) for i in range(len(self.groups))])
        if rc == _TOO_LONG:
            who = requests[int(short[0])]
            raise SequenceTooLong(
                f"request {who!r} would pass position {self.max_positions}, the most the model "
                f"was built for (it is at {self.position(who)} and brings "
                f"{list(n_new)[int(short[0])]} tokens)")
        if rc == _BAD_ARG:
            raise ValueError("a request appears twice in the batch, or a token count is negative")
        if rc != _OK:
            raise RuntimeError(f"cm_reserve failed with {rc}")

    def commit(self, request: Hashable, n_new: int, pos_advance: Optional[int] = None) -> None:
        """The forward pass over ``n_new`` tokens is done: the length advances by ``n_new``,
        the position counter by ``pos_advance`` (None: by ``n_new`` as well; the reference
        lets a model advance positions on its own, mstar/engine/cache_manager.py:777-808)."""
        if pos_advance is not None and pos_advance < 0:
            raise ValueError("pos_advance must be >= 0")
        rc = self._lib.cm_commit_positions(self._h, self._rid(request), int(n_new),
                                           -1 if pos_advance is None else int(pos_advance))
        if rc == _BAD_ARG:
            raise ValueError(f"commit of {n_new} tokens for {request!r} without reserved pages")
        if rc != _OK:
            raise RuntimeError(f"cm_commit failed with {rc}")

    # -- queries ----------------------------------------------------------
    def length(self, request: Hashable) -> int:
        return int(self._lib.cm_len(self._h, self._rid(request)))

    def position(self, request: Hashable) -> int:
        """Position id of the request's next token; equal to ``length`` unless a commit
        advanced the two differently or ``set_position`` moved it."""
        return int(self._lib.cm_position(self._h, self._rid(request)))

    def set_position(self, request: Hashable, position: int) -> None:
        rc = self._lib.cm_set_position(self._h, self._rid(request), int(position))
        if rc != _OK:
            raise ValueError(f"cannot set the position counter of {request!r} to {position}")

    def slot(self, request: Hashable) -> int:
        return int(self._lib.cm_slot(self._h, self._rid(request)))

    def free_pages(self, group: int = 0) -> int:
        return int(self._lib.cm_free_pages(self._h, group))

    def free_slots(self) -> int:
        return int(self._lib.cm_free_slots(self._h))

    def num_requests(self) -> int:
        return int(self._lib.cm_num_requests(self._h))

    def block_table(self, request: Hashable, group: int = 0) -> list[int]:
        rid = self._rid(request)
        n = self._lib.cm_block_table(self._h, rid, group, _i32([0]), 0)
        if n < 0:
            raise RuntimeError(f"cm_block_table failed with {n}")
        buf = _i32([0] * max(1, n))
        self._lib.cm_block_table(self._h, rid, group, buf, n)
        return [int(buf[i]) for i in range(n)]

    def check(self) -> int:
        """Number of violated invariants (0 when no page or slot is lost, held
        twice or free twice)."""
        return int(self._lib.cm_check(self._h))

    # -- per-step index arrays ---------------------------------------------
    def batch_widths(self, requests: Sequence[Hashable]) -> list:
        """Logical pages of the longest block table of the batch, per group."""
        rids = _i64([self._rid(r) for r in requests])
        widths_c = _i32([0] * max(1, len(self.groups)))
        rc = self._lib.cm_batch_widths(self._h, len(requests), rids, widths_c)
        if rc != _OK:
            raise RuntimeError(f"cm_batch_widths failed with {rc}")
        return [int(widths_c[g]) for g in range(len(self.groups))]

    def fill_batch(self, requests: Sequence[Hashable], n_new: Sequence[int],
                   extra: Sequence[tuple] = (), alloc=None, *, widths=None,
                   pad_entries: int = 0, pad_page: int = 0, pad_slot: int = 0) -> BatchIndex:
        """Index arrays for a batch whose pages are reserved, packed in one int32
        buffer so that one copy brings them to the device.  ``extra``: further
        (name, length) sections the caller fills itself (token ids, wanted rows);
        ``alloc(n)`` returns the int32 array to pack into (pinned memory).

        For batches of a fixed shape (CUDA graphs): ``widths`` fixes the row length
        of each group's block table, and ``pad_entries`` appends entries of one token
        each at position 0 whose only page is ``pad_page`` and whose slot is
        ``pad_slot`` (a page and a slot that no request ever owns)."""
        n = len(requests)
        rids = _i64([self._rid(r) for r in requests])
        counts = [int(c) for c in n_new]
        if widths is None:
            widths = [max(1, w) for w in self.batch_widths(requests)]
        else:
            widths = [int(w) for w in widths]
        real_total = sum(counts)
        n_all = n + int(pad_entries)
        total = real_total + int(pad_entries)
        offsets: dict = {}
        cursor = 0

        def take(name: str, length: int) -> None:
            nonlocal cursor
            offsets[name] = (cursor, length)
            cursor = _round4(cursor + length)

        take("token_req", total)
        take("positions", total)
        take("cache_pos", total)
        take("qo_indptr", n_all + 1)
        take("kv_len", n_all)
        take("slots", n_all)
        for g, w in enumerate(widths):
            take(f"table{g}", n_all * w)
        for name, length in extra:
            take(name, int(length))
        size = max(cursor, 4)
        if alloc is None:
            packed = np.zeros(size, dtype=np.int32)
        else:
            packed = alloc(size)
            if packed.dtype != np.int32 or packed.size < size:
                raise ValueError(f"index buffer too small: need {size} int32")
            packed = packed[:size]

        def view(name: str) -> np.ndarray:
            o, length = offsets[name]
            return packed[o:o + length]

        pi32 = ctypes.POINTER(ctypes.c_int)

        def ptr(arr: np.ndarray):
            return arr.ctypes.data_as(pi32)

        tables = [view(f"table{g}").reshape(n_all, w) for g, w in enumerate(widths)]
        table_ptrs = (pi32 * max(1, len(tables)))(*[ptr(t) for t in tables])
        rc = self._lib.cm_fill_batch(
            self._h, n, rids, _i32(counts), ptr(view("token_req")), ptr(view("positions")),
            ptr(view("cache_pos")), ptr(view("qo_indptr")), ptr(view("kv_len")),
            ptr(view("slots")), table_ptrs, _i32(widths))
        if rc == _BAD_ARG:
            raise ValueError("fill_batch before reserve (a request lacks pages for its "
                             "tokens), or a block table wider than the fixed width")
        if rc != _OK:
            raise RuntimeError(f"cm_fill_batch failed with {rc}")
        if pad_entries:
            view("token_req")[real_total:] = np.arange(n, n_all, dtype=np.int32)
            view("positions")[real_total:] = 0
            view("cache_pos")[real_total:] = 0
            view("qo_indptr")[n + 1:] = real_total + np.arange(1, pad_entries + 1, dtype=np.int32)
            view("kv_len")[n:] = 1
            view("slots")[n:] = pad_slot
            for g, t in enumerate(tables):
                t[n:, :] = -1
                t[n:, 0] = pad_page[g] if isinstance(pad_page, (list, tuple)) else pad_page
        return BatchIndex(packed=packed, num_tokens=total, num_entries=n_all,
                          token_req=view("token_req"), positions=view("positions"),
                          cache_pos=view("cache_pos"), qo_indptr=view("qo_indptr"),
                          kv_len=view("kv_len"), slots=view("slots"), tables=tables,
                          offsets=offsets)
