"""Rotary position encoding with the llama3 frequency scaling.

Unscaled: inv_freq_j = theta^(-2j/rotary_dim), angle = position * inv_freq_j,
(x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin) on split-half pairs
(mstar/utils/attention.py:224-253).  The reference passes the llama3 parameters
(factor, low/high frequency factors, original context length) to a library call
(mstar/engine/cache_manager.py:752-759, mstar/model/components/distributed/
attention.py:122-136) and never writes the rule down; it is, per frequency with
wavelength L = 2 pi / inv_freq and original context C:
    L < C / high_freq_factor  -> unchanged
    L > C / low_freq_factor   -> inv_freq / factor
    otherwise s = (C / L - low) / (high - low),
              inv_freq' = (1 - s) * inv_freq / factor + s * inv_freq.
The table of frequencies is computed once on the host in double precision and
rounded to float; angles are float(position) * inv_freq in float on the device.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import Runtime
from .registry import register_part


def rope_inverse_frequencies(spec) -> list:
    """``rotary_dim / 2`` frequencies as Python floats (double precision)."""
    half = spec.rotary_dim // 2
    freqs = [spec.theta ** (-(2.0 * j) / spec.rotary_dim) for j in range(half)]
    sc = spec.scaling
    if sc is None:
        return freqs
    if sc.rope_type != "llama3":
        raise ValueError(f"rope scaling {sc.rope_type!r} is not supported")
    low_wavelen = sc.original_max_position_embeddings / sc.low_freq_factor
    high_wavelen = sc.original_max_position_embeddings / sc.high_freq_factor
    out = []
    for f in freqs:
        wavelen = 2.0 * math.pi / f
        if wavelen < high_wavelen:
            out.append(f)
        elif wavelen > low_wavelen:
            out.append(f / sc.factor)
        else:
            smooth = (sc.original_max_position_embeddings / wavelen - sc.low_freq_factor) / (
                sc.high_freq_factor - sc.low_freq_factor)
            out.append((1.0 - smooth) * f / sc.factor + smooth * f)
    return out


class RotaryEncoding:
    """Position part of kind "rope".  It is applied by the fused kernel that also
    writes keys and values into their pages."""

    @classmethod
    def param_specs(cls, spec) -> dict:
        return {}

    def __init__(self, spec, params: dict, runtime: Runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and in "
                             f"(0, head_dim={spec.head_dim}]")
        self.spec = spec
        self.inv_freq = torch.tensor(rope_inverse_frequencies(spec), dtype=torch.float64).to(
            torch.float32).to(runtime.device)

    def apply(self, qkv, ctx, kv_cache, block_table, page_size, num_heads, num_kv_heads):
        ops.rope_kv_write(qkv, ctx.positions, ctx.cache_pos, ctx.token_req, block_table,
                          self.inv_freq, kv_cache, num_heads, num_kv_heads, self.spec.head_dim,
                          self.spec.rotary_dim, self.spec.interleaved, page_size)

    def project_and_apply(self, x, w_qkv, ctx, kv_cache, block_table, page_size, num_heads,
                          num_kv_heads):
        """Optional entry of a position part: the mixer's first product together with
        ``apply``, where one kernel does both (a few decoded tokens, split-half pairs over
        the whole head).  Returns the rotated queries [tokens, num_heads * head_dim], keys
        and values being in the cache; or None, and the mixer takes the two steps."""
        s = self.spec
        if s.interleaved or s.rotary_dim != s.head_dim:
            return None
        return ops.qkv_rope_write(x, w_qkv, ctx.positions, ctx.cache_pos, ctx.token_req,
                                  block_table, self.inv_freq, kv_cache, num_heads, num_kv_heads,
                                  s.head_dim, page_size, static_weights=True)


class NoPositionEncoding:
    """Position part of kind "none": keys and values are written as they are."""

    @classmethod
    def param_specs(cls, spec) -> dict:
        return {}

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec

    def apply(self, qkv, ctx, kv_cache, block_table, page_size, num_heads, num_kv_heads):
        ops.rope_kv_write(qkv, ctx.positions, ctx.cache_pos, ctx.token_req, block_table, None,
                          kv_cache, num_heads, num_kv_heads, self.spec.head_dim, 0, False,
                          page_size)


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
