"""Architecture-neutral description of a decoder: the specs that parts are built from.

A model configuration (for instance ``LlamaConfig``) is turned into a
``ModelLayout``: one ``BlockSpec`` per set of layer weights, each naming its
mixer, feed-forward, norms and their arrangement, and a run order that says
which block runs when and which cache it uses.  The engine only ever sees
these specs, so nothing below the configuration knows which model it is in.

Every spec carries a ``kind`` string.  ``mstar_b200.parts.registry`` maps
``(category, kind)`` to the class that implements it; a new mixer,
feed-forward, norm, position encoding or block arrangement is a new spec
dataclass plus one ``register_part`` call.

The reference builds its decoder layer from interchangeable modules in the
same spirit (mstar/model/components/decoder_layer.py:45-56) but takes the
sizes from a hard-coded dataclass (mstar/model/orpheus/config.py:4-53).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass(frozen=True)
class RopeScalingSpec:
    """Frequency-dependent scaling of rotary frequencies ("llama3" rule)."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    kind "rope": rotary embedding over the first ``rotary_dim`` features of
    each head, pairs ``(j, j + rotary_dim/2)`` unless ``interleaved``.
    kind "none": nothing is applied.
    """

    kind: str = "rope"
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    scaling: Optional[RopeScalingSpec] = None
    interleaved: bool = False


@dataclass(frozen=True)
class NormSpec:
    """kind "rmsnorm": ``x * rsqrt(mean(x^2) + eps) * (weight + weight_offset)``."""

    kind: str = "rmsnorm"
    size: int = 0
    eps: float = 1e-6
    weight_offset: float = 0.0


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window``: None keeps every key; ``W`` lets a token at position ``p``
    see keys ``p-W+1 .. p``.  ``shares_kv``: the layer has no key/value
    projections and reads the cache written by an earlier layer.
    ``scale``: None means ``head_dim ** -0.5``.
    """

    kind: str = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    position: PositionSpec = field(default_factory=PositionSpec)
    window: Optional[int] = None
    scale: Optional[float] = None
    shares_kv: bool = False


@dataclass(frozen=True)
class GatedMLPSpec:
    """``down(act(gate(x)) * up(x))`` with a fused ``[gate; up]`` matrix."""

    kind: str = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class EmbeddingSpec:
    """kind "table": the residual starts as ``table[token] * multiplier`` in float."""

    kind: str = "table"
    vocab_size: int = 0
    hidden_size: int = 0
    multiplier: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """kind "linear": ``logits = x W^T * logit_scale``, then ``softcap * tanh(logits /
    softcap)`` when a soft cap is given; float logits."""

    kind: str = "linear"
    vocab_size: int = 0
    hidden_size: int = 0
    logit_scale: float = 1.0
    softcap: Optional[float] = None


@dataclass(frozen=True)
class BlockSpec:
    """One set of layer weights and how its parts are wired.

    kind "prenorm": ``h += mixer(norm1(h)); h += ffn(norm2(h))``.
    ``mixer`` / ``ffn`` are any registered spec; they may differ from block
    to block within one model.
    """

    kind: str
    mixer: object
    ffn: object
    norm1: NormSpec
    norm2: NormSpec


@dataclass(frozen=True)
class RunEntry:
    """One position in the execution order.

    ``block``: index into ``ModelLayout.blocks`` (a block may appear twice,
    its weights are then shared).  ``cache``: index of the cache this run
    reads and writes; by default every run has its own.  A run whose mixer
    ``shares_kv`` names the cache of the earlier run it reads.
    """

    block: int
    cache: int


@dataclass(frozen=True)
class ModelLayout:
    vocab_size: int
    hidden_size: int
    blocks: Sequence[BlockSpec]
    order: Sequence[RunEntry]
    final_norm: NormSpec
    tie_word_embeddings: bool = False
    # position ids run over [0, max_positions); None: no limit is known
    max_positions: Optional[int] = None
    # what turns token ids into the residual and normed rows into logits; None: a plain
    # table and a plain linear head of the layout's sizes
    embedding: Optional[object] = None
    head: Optional[object] = None

    def embedding_spec(self):
        return self.embedding or EmbeddingSpec(vocab_size=self.vocab_size,
                                               hidden_size=self.hidden_size)

    def head_spec(self):
        return self.head or HeadSpec(vocab_size=self.vocab_size, hidden_size=self.hidden_size)

    def num_caches(self) -> int:
        return 1 + max((e.cache for e in self.order), default=-1)

    def validate(self) -> None:
        if not self.blocks:
            raise ValueError("a model layout needs at least one block")
        owners: dict[int, int] = {}
        for pos, entry in enumerate(self.order):
            if not 0 <= entry.block < len(self.blocks):
                raise ValueError(f"run order entry {pos} names block {entry.block}, "
                                 f"but the layout has {len(self.blocks)} blocks")
            mixer = self.blocks[entry.block].mixer
            if getattr(mixer, "shares_kv", False):
                if entry.cache not in owners:
                    raise ValueError(f"run order entry {pos} reads cache {entry.cache} "
                                     "before any earlier entry has written it")
            else:
                if entry.cache in owners:
                    raise ValueError(f"cache {entry.cache} is written by run order entries "
                                     f"{owners[entry.cache]} and {pos}")
                owners[entry.cache] = pos
        missing = sorted(set(range(self.num_caches())) - set(owners))
        if missing:
            raise ValueError(f"caches {missing} are never written")
