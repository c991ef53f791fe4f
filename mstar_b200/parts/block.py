"""Block arrangements: how a mixer, a feed-forward and norms are wired.

"prenorm" is the reference's DecoderLayer (mstar/model/components/decoder_layer.py:
58-71): h += mixer(norm1(h)); h += ffn(norm2(h)).  The two adds are not separate
passes: each part's output stays pending on the residual stream and the next norm
(the next block's norm1, or the final norm) adds it in float while normalising.
"""
from __future__ import annotations

from .base import ResidualStream, Runtime
from .registry import build_part, part_class, register_part


def _sub(params: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in params.items() if k.startswith(p)}


class PreNormBlock:
    SUBPARTS = (("norm1", "norm"), ("mixer", "mixer"), ("norm2", "norm"), ("ffn", "ffn"))

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls.SUBPARTS:
            sub = getattr(spec, name)
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.norm1 = build_part("norm", spec.norm1, _sub(params, "norm1"), runtime)
        self.mixer = build_part("mixer", spec.mixer, _sub(params, "mixer"), runtime)
        self.norm2 = build_part("norm", spec.norm2, _sub(params, "norm2"), runtime)
        self.ffn = build_part("ffn", spec.ffn, _sub(params, "ffn"), runtime)
        # replayable as part of a captured decode step only if every sub-part says so itself
        self.graph_safe = all(getattr(p, "graph_safe", False) is True
                              for p in (self.norm1, self.mixer, self.norm2, self.ffn))

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.norm1.add_norm(stream)
        stream.push(self.mixer.forward(x, ctx, cache))
        y = self.norm2.add_norm(stream)
        stream.push(self.ffn.forward(y, ctx))


register_part("block", "prenorm", PreNormBlock)
