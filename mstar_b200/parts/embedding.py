"""Token embedding and LM head parts: the two ends of the residual stream.

"table": h0 = E[ids] (mstar/model/orpheus/components/language_model.py:61-66, no scaling
there; ``multiplier`` serves architectures that scale the rows), written as the float
residual.  "linear": logits = x W^T without bias (language_model.py:95-101), float, with an
optional scale and soft cap.  A tied head is the same tensor under two parameter names;
the checkpoint map says so, the parts do not know.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import Runtime, StepContext
from .registry import register_part


class TokenEmbedding:
    graph_safe = True

    @classmethod
    def param_specs(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab_size, spec.hidden_size), role="table")}

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.weight = params["weight"]

    def forward(self, token_ids: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """Float residual [tokens, hidden]; tokens that only the device holds come through
        ``ctx.token_source``."""
        return ops.embed_rows(self.weight, token_ids, source=ctx.token_source,
                              scale=self.spec.multiplier)


class LinearHead:
    graph_safe = True

    @classmethod
    def param_specs(cls, spec) -> dict:
        return {"weight": ParamSpec((spec.vocab_size, spec.hidden_size))}

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.weight = params["weight"]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Float logits [rows, vocab] of normed rows ``x``."""
        logits = ops.linear(x, self.weight, out_dtype=torch.float32, static_weights=True)
        if self.spec.logit_scale != 1.0 or self.spec.softcap:
            ops.scale_softcap(logits, self.spec.logit_scale, self.spec.softcap)
        return logits


register_part("embedding", "table", TokenEmbedding)
register_part("head", "linear", LinearHead)
