"""Grouped-query attention mixer over the paged cache.

Order of operations as in the reference (mstar/model/components/distributed/
attention.py:98-110, 138-149): one fused QKV product, split [q | k | v], position
encoding on q and k, write of k and v into the cache, attention, output product.
Query head i uses key/value head i // (num_heads / num_kv_heads); scores are scaled
by head_dim ** -0.5 unless the spec says otherwise; the mask is causal and aligned
to the end of the key sequence, optionally limited to a window of keys.

A layer with ``shares_kv`` has only the query and output products and reads the
cache that an earlier layer wrote.
"""
from __future__ import annotations

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, KVNeed, LayerCache, Runtime, StepContext
from .registry import build_part, register_part


class Attention:
    # everything the forward pass does depends on the step's device arrays and on host
    # values that are fixed for a batch shape, so a decode step can be replayed as a
    # CUDA graph
    graph_safe = True

    @classmethod
    def param_specs(cls, spec) -> dict:
        q_rows = spec.num_heads * spec.head_dim
        kv_rows = spec.num_kv_heads * spec.head_dim
        if spec.shares_kv:
            first = {"q.weight": ParamSpec((q_rows, spec.hidden_size))}
        else:
            first = {"qkv.weight": ParamSpec((q_rows + 2 * kv_rows, spec.hidden_size))}
        first["o.weight"] = ParamSpec((spec.hidden_size, q_rows))
        return first

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kv=KVNeed(num_kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                                   window=spec.window))

    def __init__(self, spec, params: dict, runtime: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads {spec.num_heads} is not a multiple of num_kv_heads "
                             f"{spec.num_kv_heads}")
        if spec.head_dim % 16:
            raise ValueError(f"head_dim {spec.head_dim} must be a multiple of 16")
        self.spec = spec
        self.runtime = runtime
        self.w_in = params["q.weight"] if spec.shares_kv else params["qkv.weight"]
        self.w_out = params["o.weight"]
        self.position = build_part("position", spec.position, {}, runtime)
        # a position part may offer the first product and its own work as one call
        self._fused_projection = getattr(self.position, "project_and_apply", None)
        self.scale = spec.scale if spec.scale is not None else spec.head_dim ** -0.5

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        write_heads = 0 if s.shares_kv else s.num_kv_heads
        qkv = None
        if self._fused_projection is not None and not s.shares_kv:
            # queries only, [tokens, heads * head_dim]; keys and values are in the cache
            qkv = self._fused_projection(x, self.w_in, ctx, cache.kv, cache.block_table,
                                         cache.page_size, s.num_heads, write_heads)
        if qkv is None:
            qkv = ops.linear(x, self.w_in, static_weights=True)
            self.position.apply(qkv, ctx, None if s.shares_kv else cache.kv, cache.block_table,
                                cache.page_size, s.num_heads, write_heads)
        out = qkv.new_empty((ctx.num_tokens, s.num_heads * s.head_dim))
        self.attend(qkv, out, ctx, cache)
        return ops.linear(out, self.w_out, static_weights=True)

    def attend(self, qkv, out, ctx: StepContext, cache: LayerCache) -> None:
        """bfloat16 with a head size the tensor-core kernels take: single-token entries
        (they come first in the batch) go to the split-K decode kernel, prompt portions
        to the prefill kernel.  Everything else, float32 included, runs the generic
        kernel."""
        s = self.spec
        if ops.fast_attention_supported(qkv.dtype, s.num_heads, s.num_kv_heads, s.head_dim):
            nd = ctx.num_decode
            if nd:
                ops.paged_decode_attention(
                    qkv, qkv.stride(0), out, cache.kv, cache.block_table, ctx.token_req,
                    ctx.cache_pos, nd, s.num_heads, s.num_kv_heads, s.head_dim,
                    cache.page_size, s.window or 0, self.scale, max(ctx.kv_lens[:nd]),
                    static_keys=True)
            if ctx.num_entries > nd:
                ops.paged_prefill_attention(
                    qkv, qkv.stride(0), out, cache.kv, cache.block_table, ctx.qo_indptr,
                    ctx.kv_len, nd, ctx.num_entries - nd, max(ctx.q_lens[nd:]), s.num_heads,
                    s.num_kv_heads, s.head_dim, cache.page_size, s.window or 0, self.scale)
            return
        ops.paged_attention_generic(
            qkv, qkv.stride(0), out, cache.kv, cache.block_table, ctx.token_req, ctx.cache_pos,
            ctx.num_tokens, s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size,
            s.window or 0, self.scale)


register_part("mixer", "attention", Attention)
