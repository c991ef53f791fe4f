"""A model instance: embedding, blocks in their run order, final norm, LM head.

Built from a ``ModelLayout`` alone; which architecture produced the layout is
not known here.  The forward pass follows the reference's language model
(mstar/model/orpheus/components/language_model.py:72-83: embed, every layer, final
norm); the two ends, token ids to residual and normed rows to logits, are parts of their
own, so that a scaled embedding or a capped head is a spec and not an edit here.  The row
selection is moved before the final norm: only rows whose logits
are wanted are normalised and multiplied by the head (the reference norms all rows
and then selects the last one of each request, mstar/model/orpheus/submodules.py:
225-231).
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Sequence

import torch

from .. import ops
from ..config.base import ModelConfig
from ..config.layout import ModelLayout
from ..config.registry import get_architecture, load_config
from ..parts.base import CacheNeed, ResidualStream, Runtime, StepContext
from ..parts.registry import build_part, part_class
from ..weights.loader import load_parameters
from ..weights.names import ParamSpec


def model_param_specs(layout: ModelLayout) -> dict:
    """Engine parameter names and shapes of a layout (no GPU needed)."""
    specs = {}
    embedding = layout.embedding_spec()
    for local, ps in part_class("embedding", embedding).param_specs(embedding).items():
        specs[f"embed.{local}"] = ps
    for i, block in enumerate(layout.blocks):
        for local, ps in part_class("block", block).param_specs(block).items():
            specs[f"blocks.{i}.{local}"] = ps
    norm_cls = part_class("norm", layout.final_norm)
    for local, ps in norm_cls.param_specs(layout.final_norm).items():
        specs[f"final_norm.{local}"] = ps
    head = layout.head_spec()
    for local, ps in part_class("head", head).param_specs(head).items():
        specs[f"head.{local}"] = ps
    return specs


def cache_needs(layout: ModelLayout) -> list:
    """What each cache (by id) has to hold, from the mixer that writes it."""
    needs: list = [None] * layout.num_caches()
    for entry in layout.order:
        block = layout.blocks[entry.block]
        if getattr(block.mixer, "shares_kv", False):
            continue
        need = part_class("block", block).cache_need(block)
        needs[entry.cache] = need if need is not None else CacheNeed()
    return needs


def _sub(params: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in params.items() if k.startswith(p)}


class Model:
    def __init__(self, config: Optional[ModelConfig], layout: ModelLayout, params: dict,
                 runtime: Runtime):
        layout.validate()
        self.config = config
        self.layout = layout
        self.runtime = runtime
        self.params = params
        self.embedding = build_part("embedding", layout.embedding_spec(), _sub(params, "embed"),
                                    runtime)
        self.head = build_part("head", layout.head_spec(), _sub(params, "head"), runtime)
        self.blocks = [build_part("block", spec, _sub(params, f"blocks.{i}"), runtime)
                       for i, spec in enumerate(layout.blocks)]
        self.final_norm = build_part("norm", layout.final_norm, _sub(params, "final_norm"),
                                     runtime)
        self.cache_needs = cache_needs(layout)
        # a decode step may be captured as a CUDA graph only if every block says that its
        # forward pass reads nothing per-step from the host; a block that says nothing is
        # taken as unsafe
        self.graph_safe = all(getattr(p, "graph_safe", False) is True
                              for p in (self.embedding, self.head, self.final_norm, *self.blocks))

    @property
    def vocab_size(self) -> int:
        return self.layout.vocab_size

    @property
    def max_positions(self) -> Optional[int]:
        """Positions the model was built for (its layout says; None: no limit known)."""
        return self.layout.max_positions

    def parameter_bytes(self) -> int:
        seen, total = set(), 0
        for t in self.params.values():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, storage,
                block_tables: Sequence[torch.Tensor],
                want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """Run the tokens of one step; return float logits [len(want_rows), vocab]."""
        stream = ResidualStream(self.embedding.forward(token_ids, ctx))
        for entry in self.layout.order:
            self.blocks[entry.block].forward(stream, ctx, storage.layer_cache(entry.cache,
                                                                               block_tables))
        if want_rows is None or want_rows.numel() == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32,
                               device=self.runtime.device)
        rows = ops.gather_add_rows(stream.h, stream.take_delta(), want_rows)
        x = self.final_norm.norm_rows(rows)
        return self.head.forward(x)


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        out = dtype
    else:
        names = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                 "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}
        if dtype not in names:
            raise ValueError(f"dtype {dtype!r} is not supported (bfloat16, float32)")
        out = names[dtype]
    if out not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype {out} is not supported (bfloat16, float32)")
    return out


def load_model(source, dtype="bfloat16", device="cuda:0", *, config: Optional[ModelConfig] = None,
               tensors=None) -> Model:
    """Build a model from a folder (config.json + safetensors).  ``config`` and
    ``tensors`` (checkpoint name -> tensor) replace the folder's files when given."""
    dt = resolve_dtype(dtype)
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("mstar_b200 runs on CUDA devices only (there is no CPU path); "
                           f"got device {device!r}")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available: mstar_b200 needs an NVIDIA B200 "
                           "(sm_100a) GPU")
    if config is None:
        config = load_config(source)
    layout = config.layout()
    arch = get_architecture(config.architecture)
    specs = model_param_specs(layout)
    cmap = arch.checkpoint_map(config, layout)
    params = load_parameters(tensors if tensors is not None else Path(source), specs, cmap,
                             dt, dev)
    return Model(config, layout, params, Runtime(dtype=dt, device=dev))
