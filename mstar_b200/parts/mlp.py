"""Gated feed-forward: down(act(gate(x)) * up(x)) with one fused [gate; up] matrix
(mstar/model/components/distributed/mlp.py:78-81; gate is shard 0, up shard 1)."""
from __future__ import annotations

from .. import ops
from ..weights.names import ParamSpec
from .base import Runtime
from .registry import register_part


class GatedMLP:
    graph_safe = True       # nothing per-step is read from the host

    @classmethod
    def param_specs(cls, spec) -> dict:
        return {
            "gate_up.weight": ParamSpec((2 * spec.intermediate_size, spec.hidden_size)),
            "down.weight": ParamSpec((spec.hidden_size, spec.intermediate_size)),
        }

    def __init__(self, spec, params: dict, runtime: Runtime):
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp activation {spec.activation!r} has no kernel (silu has)")
        self.spec = spec
        self.runtime = runtime
        self.gate_up = params["gate_up.weight"]
        self.down = params["down.weight"]

    def forward(self, x, ctx):
        return ops.linear(ops.gated_up(x, self.gate_up, static_weights=True), self.down,
                          static_weights=True)


register_part("ffn", "gated_mlp", GatedMLP)
