"""What parts and the step function share: the runtime, the step context, the
residual stream and the description of a mixer's cache needs."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class KVNeed:
    """Keys and values in pages: [pages, 2, num_kv_heads, page_size, head_dim].
    ``window`` None keeps every key; W keeps the last W."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one ``shape`` tensor per state slot,
    zeroed when a request takes the slot."""

    shape: tuple
    dtype: str = "float32"


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


@dataclass
class Runtime:
    """Compute dtype and device of a model instance."""

    dtype: torch.dtype
    device: torch.device


@dataclass
class LayerCache:
    """The cache of one run-order entry, as its mixer sees it."""

    kv: Optional[torch.Tensor] = None           # [pages, 2, kv_heads, page_size, head_dim]
    page_size: int = 0
    block_table: Optional[torch.Tensor] = None  # int32 [entries, width] of the cache's group
    state: Optional[torch.Tensor] = None        # [slots, *shape]


@dataclass
class StepContext:
    """Index arrays of one step on the device (int32) plus host copies.

    Tokens are packed entry after entry.  ``token_req[t]`` is the entry of token
    t, ``positions[t]`` its position id, ``cache_pos[t]`` the index of its key in
    the request's key sequence (kept apart from the position id, as the reference
    keeps position_id_start apart from seq_len, mstar/engine/kv_store.py:112-116).
    """

    num_tokens: int
    num_entries: int
    token_req: torch.Tensor
    positions: torch.Tensor
    cache_pos: torch.Tensor
    qo_indptr: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    # host copies (python lists) for parts that plan on the host
    q_lens: list = field(default_factory=list)
    kv_lens: list = field(default_factory=list)
    host_slots: list = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    # entries [0, num_decode) bring exactly one token each (tokens [0, num_decode))
    num_decode: int = 0
    # (src, prev) or None: where src[t] >= 0, token t is prev[src[t]], a token that the step
    # before sampled and that only the device holds yet (int32 tensors)
    token_source: Optional[tuple] = None
    extras: dict = field(default_factory=dict)


class ResidualStream:
    """The float residual ``h`` and the not-yet-added output ``delta`` of the last
    part.  Norm parts fold ``h += delta`` into the normalisation that follows, so
    the residual sum is a 32-bit sum and costs no pass of its own."""

    def __init__(self, h: torch.Tensor):
        assert h.dtype == torch.float32
        self.h = h
        self.delta: Optional[torch.Tensor] = None

    def push(self, delta: torch.Tensor) -> None:
        if self.delta is not None:
            raise RuntimeError("a part's output was pushed before the previous one was added")
        self.delta = delta

    def take_delta(self) -> Optional[torch.Tensor]:
        d, self.delta = self.delta, None
        return d
