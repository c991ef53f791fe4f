"""Random-weights mode: make a model folder from a configuration and a seed.

The reference has no such mode (its tests use real checkpoints).  Tensors are
drawn under their checkpoint names (unfused q/k/v, gate/up), so that loading
the folder exercises the same packing path as a real checkpoint.  Values are
rounded to bfloat16 before they are stored, whatever the storage dtype, so a
32-bit and a bfloat16 run of the same folder use identical weights.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping, Optional

import torch

from ..config.base import ModelConfig
from ..config.registry import get_architecture
from .names import ParamSpec


def checkpoint_tensor_shapes(config: ModelConfig, param_specs: Mapping[str, ParamSpec]) -> dict:
    """``{checkpoint name: (shape, ParamSpec of the parameter it fills)}``; tensors
    that the map marks optional (a tied head) are left out."""
    arch = get_architecture(config.architecture)
    cmap = arch.checkpoint_map(config, config.layout())
    out = {}
    for src in cmap.sources:
        if src.name in cmap.optional:
            continue
        spec = param_specs[src.param]
        out[src.name] = ((src.rows,) + tuple(spec.shape[1:]), spec)
    return out


def random_checkpoint(config: ModelConfig, seed: int, *, std: float = 0.02,
                      norm_noise: float = 0.0, dtype: torch.dtype = torch.bfloat16,
                      vector_dtype: Optional[torch.dtype] = None,
                      device: str | torch.device = "cpu") -> dict:
    """Draw every checkpoint tensor.  Matrices and tables ~ N(0, std); norm
    weights 1 + N(0, norm_noise).  ``vector_dtype`` stores norm weights in
    another dtype than the matrices (float32 exercises the "stays 32-bit" rule)."""
    from ..engine.model import model_param_specs

    specs = model_param_specs(config.layout())
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: dict = {}
    for name, (shape, spec) in checkpoint_tensor_shapes(config, specs).items():
        if spec.role == "int_table":
            t = torch.randint(0, 2 ** 15, shape, generator=gen, device=device, dtype=torch.int32)
            out[name] = t
            continue
        store = dtype
        if spec.init == "ones":
            t = torch.ones(shape, dtype=torch.float32, device=device)
            if norm_noise:
                t += norm_noise * torch.randn(shape, generator=gen, device=device,
                                              dtype=torch.float32)
            store = vector_dtype or dtype
        elif spec.init == "zeros":
            t = torch.zeros(shape, dtype=torch.float32, device=device)
        else:
            t = std * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        out[name] = t.to(torch.bfloat16).to(store)
    return out


def write_model_folder(folder: str | Path, config: ModelConfig, seed: int, *,
                       tensors: Optional[Mapping] = None, **kwargs) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a random model; ``tensors``
    (checkpoint name -> tensor) are written instead of freshly drawn ones if given."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    if tensors is None:
        tensors = random_checkpoint(config, seed, **kwargs)
    raw = config.to_dict()
    (folder / "config.json").write_text(json.dumps(raw, indent=2, sort_keys=True) + "\n")
    save_file({k: v.contiguous().cpu() for k, v in tensors.items()},
              str(folder / "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder
