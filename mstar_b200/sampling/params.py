"""Per-request sampling options, in the reference's names and meanings
(mstar/utils/sampling.py:207-226; per-request overrides of temperature, top_p,
repetition_penalty and ignore_eos, mstar/model/orpheus/orpheus_model.py:362-381;
max_output_tokens, mstar/model/base.py:30; seed from the request id unless given,
mstar/conductor/conductor.py:51-63, 621-622)."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.6          # 0 = greedy
    top_k: int = 0                    # 0 = off
    top_p: float = 1.0                # 1 = off
    repetition_penalty: float = 1.0   # 1 = off; applies to tokens generated so far
    ignore_eos: bool = False          # decode to max_output_tokens whatever is sampled
    max_output_tokens: int = 2048
    seed: Optional[int] = None        # None: derived from the request id

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if self.max_output_tokens < 1:
            raise ValueError(f"max_output_tokens must be >= 1, got {self.max_output_tokens}")


def seed_from_request_id(request_id: str) -> int:
    """Stable 32-bit seed of a request id: first four bytes of its MD5, little-endian
    (the reference's rule, mstar/conductor/conductor.py:51-63)."""
    digest = hashlib.md5(str(request_id).encode("utf-8")).digest()
    return int.from_bytes(digest[:4], "little")
