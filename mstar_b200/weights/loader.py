"""Load engine parameters from safetensors by checkpoint tensor name.

Sources, as the reference accepts them (mstar/model/loader/base.py:195-223,
mstar/model/loader/iterators.py:45-89): a folder with ``model.safetensors``, or
with ``model.safetensors.index.json`` and its shards, or a single file.

What differs from the reference is deliberate: every problem (missing tensors,
unexpected tensors, wrong shapes) is collected and raised as ONE error, whereas
the reference silently ignores unknown keys and never detects a missing
parameter (base.py:136-145).

Dtypes: with ``dtype=bfloat16`` floating tensors are kept in bfloat16, except
that a tensor the checkpoint stores in 32-bit stays in 32-bit; integer tensors
become int32.  With ``dtype=float32`` every floating tensor is widened to
float32 (bfloat16 values are exact in float32).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping, Optional

import torch

from .names import CheckpointMap, ParamSpec


class WeightsError(RuntimeError):
    """The checkpoint does not fit the model; the message lists every problem."""

    def __init__(self, where: str, missing: list, unexpected: list, wrong_shape: list,
                 other: Optional[list] = None):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other or [])
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: checkpoint {tuple(got)}, model {tuple(want)}"
                for n, got, want in self.wrong_shape))
        for msg in self.other:
            lines.append("  " + msg)
        super().__init__("\n".join(lines))


class _Checkpoint:
    """Name -> file index over one or several safetensors files (read lazily)."""

    def __init__(self, source: str | Path):
        from safetensors import safe_open

        self._memory = None
        self._handles = {}
        self.file_of: dict = {}
        if isinstance(source, Mapping):
            self._memory = dict(source)
            self.where = "<in-memory tensors>"
            return
        source = Path(source)
        self.where = str(source)
        files: list[Path]
        if source.is_file():
            files = [source]
        elif source.is_dir():
            index = source / "model.safetensors.index.json"
            single = source / "model.safetensors"
            if index.is_file():
                weight_map = json.loads(index.read_text())["weight_map"]
                files = [source / f for f in sorted(set(weight_map.values()))]
            elif single.is_file():
                files = [single]
            else:
                raise FileNotFoundError(
                    f"{source} holds neither model.safetensors nor model.safetensors.index.json")
        else:
            raise FileNotFoundError(source)
        for f in files:
            if not f.is_file():
                raise FileNotFoundError(f"checkpoint shard {f} named by the index is absent")
            handle = safe_open(str(f), framework="pt", device="cpu")
            self._handles[f] = handle
            for name in handle.keys():
                self.file_of[name] = f

    def names(self):
        if self._memory is not None:
            return self._memory.keys()
        return self.file_of.keys()

    def shape_dtype(self, name: str):
        if self._memory is not None:
            t = self._memory[name]
            return tuple(t.shape), _DTYPE_NAMES.get(t.dtype, str(t.dtype))
        sl = self._handles[self.file_of[name]].get_slice(name)
        return tuple(sl.get_shape()), str(sl.get_dtype())

    def tensor(self, name: str) -> torch.Tensor:
        if self._memory is not None:
            return self._memory[name]
        return self._handles[self.file_of[name]].get_tensor(name)


_DTYPE_NAMES = {torch.float32: "F32", torch.float64: "F64", torch.bfloat16: "BF16",
                torch.float16: "F16", torch.int32: "I32", torch.int64: "I64",
                torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}
_FLOAT32_NAMES = {"F32", "F64", "float32", "float64"}
_INT_NAMES = {"I8", "I16", "I32", "I64", "U8", "U16", "U32", "U64", "BOOL"}


def _target_dtype(spec: ParamSpec, stored: list, dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int_table" or all(s in _INT_NAMES for s in stored):
        return torch.int32
    if dtype == torch.float32:
        return torch.float32
    if any(s in _FLOAT32_NAMES for s in stored):
        return torch.float32
    return dtype


def load_parameters(source, param_specs: Mapping[str, ParamSpec],
                    cmap: CheckpointMap, dtype: torch.dtype,
                    device: torch.device | str) -> dict:
    """Return ``{engine parameter name: tensor on device}`` for every name in
    ``param_specs``; aliased parameters share storage with their target.
    ``source`` is a folder, a safetensors file, or a mapping of checkpoint names
    to tensors already in memory."""
    ckpt = _Checkpoint(source)
    by_name = cmap.by_name()
    by_param = cmap.by_param()
    ignore = cmap.ignore or (lambda n: False)

    missing: list = []
    unexpected: list = []
    wrong_shape: list = []
    other: list = []

    present = {n for n in ckpt.names() if not ignore(n)}
    for name in sorted(present):
        if name not in by_name:
            unexpected.append(name)

    aliased: dict = {}
    for param, spec in param_specs.items():
        sources = by_param.get(param, [])
        if not sources:
            other.append(f"engine parameter {param} has no checkpoint source in the "
                         "architecture's checkpoint map")
            continue
        have = [s for s in sources if s.name in present]
        if not have and param in cmap.aliases:
            aliased[param] = cmap.aliases[param]
            continue
        for s in sources:
            if s.name not in present:
                if not (s.name in cmap.optional and param in cmap.aliases and not have):
                    missing.append(s.name)
                continue
            got, _ = ckpt.shape_dtype(s.name)
            want = (s.rows,) + tuple(spec.shape[1:])
            if got != want:
                wrong_shape.append((s.name, got, want))
        covered = sum(s.rows for s in sources)
        if covered != spec.shape[0]:
            other.append(f"checkpoint map covers {covered} rows of {param}, which has "
                         f"{spec.shape[0]}")
    for name in by_name:
        if by_name[name].param not in param_specs:
            other.append(f"checkpoint map sends {name} to unknown engine parameter "
                         f"{by_name[name].param}")

    if missing or unexpected or wrong_shape or other:
        raise WeightsError(ckpt.where, sorted(missing), unexpected, wrong_shape, other)

    params: dict = {}
    kept_wide: list = []
    for param, spec in param_specs.items():
        if param in aliased:
            continue
        sources = by_param[param]
        stored = [ckpt.shape_dtype(s.name)[1] for s in sources]
        target = _target_dtype(spec, stored, dtype)
        if target == torch.float32 and dtype != torch.float32 and len(spec.shape) > 1:
            kept_wide.append(param)
        out = torch.empty(tuple(spec.shape), dtype=target, device=device)
        for s in sources:
            out.narrow(0, s.row_start, s.rows).copy_(ckpt.tensor(s.name))
        params[param] = out
    if kept_wide:
        # a tensor stored in 32 bits stays so; for a matrix that has a price worth saying
        import warnings

        shown = ", ".join(kept_wide[:4]) + (f" and {len(kept_wide) - 4} more" if len(kept_wide) > 4
                                            else "")
        warnings.warn(
            f"{len(kept_wide)} matrices of {ckpt.where} are stored in 32 bits and stay float32 "
            f"although the model runs in {str(dtype).replace('torch.', '')} ({shown}): they take "
            "twice the memory, and their products run in the true-32-bit kernel instead of the "
            "bfloat16 tensor-core kernels.  Convert the checkpoint to bfloat16 to avoid this.",
            stacklevel=2)
    for param, target_name in aliased.items():
        if target_name not in params:
            raise WeightsError(ckpt.where, [], [], [],
                               [f"{param} is tied to {target_name}, which was not loaded"])
        if tuple(params[target_name].shape) != tuple(param_specs[param].shape):
            raise WeightsError(ckpt.where, [], [],
                               [(param, params[target_name].shape, param_specs[param].shape)])
        params[param] = params[target_name]
    # A tied head whose own tensor is present as well must agree with the table.
    for param, target_name in cmap.aliases.items():
        if param in params and param not in aliased and target_name in params:
            if not torch.equal(params[param], params[target_name]):
                raise WeightsError(ckpt.where, [], [], [], [
                    f"the configuration ties {param} to {target_name}, but the checkpoint "
                    "holds both and they differ"])
            params[param] = params[target_name]
    return params
