"""Sampler: per-request options, random-number offsets and seen-token masks, and
one kernel launch per step for all rows (csrc/sampling.cu).

The reference keeps the same per-request state (config, seen mask, step offset:
mstar/utils/sampling.py:295-343) but samples with a Triton kernel plus a library
call and updates the seen masks with two launches per request (:397-412); here the
kernel that samples also marks the sampled token in the request's mask row.
"""
from __future__ import annotations

from typing import Hashable, Sequence

import torch

from .. import ops
from .params import SamplingParams, seed_from_request_id


class Sampler:
    def __init__(self, vocab_size: int, num_slots: int, device: torch.device):
        self.vocab_size = vocab_size
        self.num_slots = num_slots
        self.device = device
        self._params: dict = {}
        self._seed: dict = {}
        self._offset: dict = {}
        self._slot: dict = {}
        self._seen = None  # uint8 [num_slots, vocab], made when a request first needs it

    def add_request(self, request: Hashable, params: SamplingParams, slot: int,
                    generated: Sequence[int] = ()) -> None:
        """``generated``: tokens the request had already produced when it is admitted
        again after pre-emption; they count as seen and as drawn offsets."""
        params.validate()
        self._params[request] = params
        self._seed[request] = (params.seed if params.seed is not None
                               else seed_from_request_id(request))
        self._offset[request] = len(generated)
        self._slot[request] = slot
        if params.repetition_penalty != 1.0:
            if self._seen is None:
                self._seen = torch.zeros((self.num_slots, self.vocab_size), dtype=torch.uint8,
                                         device=self.device)
            else:
                self._seen[slot].zero_()
            self.mark_seen(request, generated)

    def remove_request(self, request: Hashable) -> None:
        for d in (self._params, self._seed, self._offset, self._slot):
            d.pop(request, None)

    def mark_seen(self, request: Hashable, tokens: Sequence[int]) -> None:
        if self._seen is None or not tokens or request not in self._slot:
            return
        if self._params[request].repetition_penalty == 1.0:
            return
        idx = torch.tensor(list(tokens), dtype=torch.long, device=self.device)
        self._seen[self._slot[request]].index_fill_(0, idx, 1)

    def sample(self, requests: Sequence[Hashable], logits: torch.Tensor) -> torch.Tensor:
        """One token per row of ``logits`` (float32 [len(requests), vocab]); int32 on
        the device.  Advances each request's random-number offset by one."""
        ps = [self._params[r] for r in requests]
        if all(p.temperature == 0 and p.repetition_penalty == 1.0 for p in ps):
            tokens = ops.argmax(logits)
        else:
            f32 = torch.tensor([[p.temperature for p in ps], [p.top_p for p in ps],
                                [p.repetition_penalty for p in ps]], dtype=torch.float32)
            i32 = torch.tensor([[p.top_k for p in ps],
                                [self._slot[r] if p.repetition_penalty != 1.0 else -1
                                 for r, p in zip(requests, ps)]], dtype=torch.int32)
            i64 = torch.tensor([[self._seed[r] for r in requests],
                                [self._offset[r] for r in requests]], dtype=torch.int64)
            f32, i32, i64 = (t.to(self.device, non_blocking=True) for t in (f32, i32, i64))
            any_k = any(p.top_k > 0 for p in ps)
            any_p = any(p.top_p < 1.0 for p in ps)
            any_pen = self._seen is not None and any(p.repetition_penalty != 1.0 for p in ps)
            tokens = ops.sample(
                logits, f32[0], top_k=i32[0] if any_k else None,
                top_p=f32[1] if any_p else None, penalty=f32[2] if any_pen else None,
                seen_mask=self._seen if any_pen else None,
                seen_rows=i32[1] if any_pen else None, seed=i64[0], offset=i64[1])
        for r in requests:
            self._offset[r] += 1
        return tokens
