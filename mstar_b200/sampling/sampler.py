"""Sampler: per-request options, random-number offsets and seen-token masks, and
one kernel launch per step for all rows (csrc/sampling.cu).

The reference keeps the same per-request state (config, seen mask, step offset:
mstar/utils/sampling.py:295-343) but samples with a Triton kernel plus a library
call and updates the seen masks with two launches per request (:397-412); here the
kernel that samples also marks the sampled token in the request's mask row.
"""
from __future__ import annotations

from typing import Hashable, Sequence

import numpy as np
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
        self._pinned = [None] * 4
        self._events = [None] * 4
        self._turn = 0

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
            # the rows' options in one pinned buffer and one copy that nothing waits for (a
            # copy from pageable memory would first wait for the step just launched)
            n = len(ps)
            host = self._staging(36 * n)
            raw = host.numpy()
            raw[0:8 * n].view(np.int64)[:] = [self._seed[r] for r in requests]
            raw[8 * n:16 * n].view(np.int64)[:] = [self._offset[r] for r in requests]
            raw[16 * n:20 * n].view(np.float32)[:] = [p.temperature for p in ps]
            raw[20 * n:24 * n].view(np.float32)[:] = [p.top_p for p in ps]
            raw[24 * n:28 * n].view(np.float32)[:] = [p.repetition_penalty for p in ps]
            raw[28 * n:32 * n].view(np.int32)[:] = [p.top_k for p in ps]
            raw[32 * n:36 * n].view(np.int32)[:] = [
                self._slot[r] if p.repetition_penalty != 1.0 else -1 for r, p in zip(requests, ps)]
            dev = torch.empty(36 * n, dtype=torch.uint8, device=self.device)
            dev.copy_(host[:36 * n], non_blocking=True)
            self._copied()
            seed, offset = dev[0:8 * n].view(torch.int64), dev[8 * n:16 * n].view(torch.int64)
            temperature = dev[16 * n:20 * n].view(torch.float32)
            top_p, penalty = (dev[20 * n:24 * n].view(torch.float32),
                              dev[24 * n:28 * n].view(torch.float32))
            top_k, seen_rows = (dev[28 * n:32 * n].view(torch.int32),
                                dev[32 * n:36 * n].view(torch.int32))
            any_k = any(p.top_k > 0 for p in ps)
            any_p = any(p.top_p < 1.0 for p in ps)
            any_pen = self._seen is not None and any(p.repetition_penalty != 1.0 for p in ps)
            tokens = ops.sample(
                logits, temperature, top_k=top_k if any_k else None,
                top_p=top_p if any_p else None, penalty=penalty if any_pen else None,
                seen_mask=self._seen if any_pen else None,
                seen_rows=seen_rows if any_pen else None, seed=seed, offset=offset)
        for r in requests:
            self._offset[r] += 1
        return tokens

    # -- pinned staging: a ring, each buffer guarded by the event after its last copy
    def _staging(self, nbytes: int) -> torch.Tensor:
        self._turn = (self._turn + 1) % len(self._pinned)
        if self._events[self._turn] is not None:
            self._events[self._turn].synchronize()
        if self._pinned[self._turn] is None or self._pinned[self._turn].numel() < nbytes:
            self._pinned[self._turn] = torch.empty(max(nbytes, 36 * 64), dtype=torch.uint8,
                                                   pin_memory=True)
        return self._pinned[self._turn]

    def _copied(self) -> None:
        event = torch.cuda.Event()
        event.record()
        self._events[self._turn] = event
