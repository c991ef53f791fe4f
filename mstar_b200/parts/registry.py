"""Registry of layer parts: (category, kind) -> class.

Categories: "mixer", "ffn", "norm", "position", "block", "embedding", "head".  A part
class offers

    param_specs(spec) -> {local name: ParamSpec}        (classmethod; no GPU needed)
    __init__(spec, params, runtime)                      params: {local name: tensor}

and, by category,

    norm      add_norm(stream) -> normed activations     (see parts/norm.py)
    position  apply(...)                                 (see parts/rope.py)
    ffn       forward(x, ctx) -> y
    mixer     cache_need(spec) -> CacheNeed              (classmethod)
              forward(x, ctx, cache) -> y
    block     sub-parts named by the spec; forward(stream, ctx, cache)
    embedding forward(token_ids, ctx) -> float residual [tokens, hidden]
    head      forward(normed rows) -> float logits [rows, vocab]

A part that may run inside a captured decode step says so with ``graph_safe = True``
(nothing per-step is read from the host); saying nothing means no.

A part never learns which model it is in: it sees its spec, its own parameters
and the step context.
"""
from __future__ import annotations

CATEGORIES = ("mixer", "ffn", "norm", "position", "block", "embedding", "head")

_PARTS: dict = {}


def register_part(category: str, kind: str, cls, *, replace: bool = False) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r} (known: {CATEGORIES})")
    key = (category, kind)
    if key in _PARTS and not replace:
        raise ValueError(f"{category} part {kind!r} is already registered")
    _PARTS[key] = cls


def unregister_part(category: str, kind: str) -> None:
    _PARTS.pop((category, kind), None)


def known_parts(category: str) -> list:
    _builtin()
    return sorted(k for c, k in _PARTS if c == category)


def part_class(category: str, spec):
    _builtin()
    kind = getattr(spec, "kind", None)
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        raise KeyError(f"no {category} part of kind {kind!r} is registered "
                       f"(known: {known_parts(category)})") from None


def build_part(category: str, spec, params: dict, runtime):
    return part_class(category, spec)(spec, params, runtime)


_done = False


def _builtin() -> None:
    global _done
    if _done:
        return
    _done = True
    from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (they register themselves)
