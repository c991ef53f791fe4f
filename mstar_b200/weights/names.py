"""Types that tie checkpoint tensor names to engine parameters.

Engine parameters have architecture-neutral names built from the layout:
``embed.weight``, ``blocks.<i>.mixer.<...>``, ``blocks.<i>.ffn.<...>``,
``blocks.<i>.norm1.weight``, ``blocks.<i>.norm2.weight``, ``final_norm.weight``,
``head.weight``.  A ``CheckpointMap`` says which rows of which parameter each
checkpoint tensor fills; fused parameters (``[q; k; v]``, ``[gate; up]``) are
several sources stacked along dim 0, the layout the reference's fused linears
use (mstar/model/components/distributed/linear.py:221-230, 145-178).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence


@dataclass(frozen=True)
class ParamSpec:
    """Shape and role of one engine parameter.

    role: "matrix" (GEMM weight), "table" (embedding), "vector" (norm weight and
    other small float tensors), "int_table" (integer lookup tables, kept int32).
    ``init``: how random-weights mode draws it: "normal" (std from the caller),
    "ones" (norm weights: 1, or 1 + noise when the caller asks for it), "zeros".
    """

    shape: tuple
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class TensorSource:
    """Checkpoint tensor ``name`` fills ``rows`` rows of ``param`` from ``row_start``."""

    name: str
    param: str
    row_start: int
    rows: int


@dataclass
class CheckpointMap:
    sources: Sequence[TensorSource]
    # engine parameter -> engine parameter it shares storage with when none of its
    # own sources is in the checkpoint (tied LM head).
    aliases: dict = field(default_factory=dict)
    # Checkpoint names that may be absent without error (sources of aliased params).
    optional: frozenset = frozenset()
    # Names that are never loaded and never reported (precomputed rotary buffers).
    ignore: Optional[Callable[[str], bool]] = None

    def by_name(self) -> dict:
        return {s.name: s for s in self.sources}

    def by_param(self) -> dict:
        out: dict = {}
        for s in self.sources:
            out.setdefault(s.param, []).append(s)
        return out
