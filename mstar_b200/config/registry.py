"""One registry from an architecture's name to everything needed to run it.

The name is ``config.json["architectures"][0]``.  The reference keys its
registry by deployment name instead and raises KeyError with the known names
(mstar/model/registry.py:8-41); the behaviour on an unknown name is kept.

Adding an architecture = one ``register_architecture`` call with
  * its ``ModelConfig`` subclass (typed config.json keys + ``layout()``),
  * a function from (config, layout) to the ``CheckpointMap`` that says which
    checkpoint tensor fills which rows of which engine parameter.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .base import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    checkpoint_map: Callable  # (ModelConfig, ModelLayout) -> weights.names.CheckpointMap


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, checkpoint_map: Callable,
                          *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    arch = Architecture(name=name, config_cls=config_cls, checkpoint_map=checkpoint_map)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    _register_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _register_builtin()
    if name not in _ARCHITECTURES:
        raise KeyError(f"Unknown architecture: {name!r}. Available: {known_architectures()}")
    return _ARCHITECTURES[name]


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    names = raw.get("architectures")
    if not names or not isinstance(names, (list, tuple)):
        raise ConfigError('config.json has no "architectures" list; cannot choose a model '
                          f"(known: {known_architectures()})")
    return get_architecture(str(names[0]))


def config_from_dict(raw: Mapping[str, Any]) -> ModelConfig:
    arch = architecture_of(raw)
    return arch.config_cls.from_dict(raw)


def load_config(folder: str | Path) -> ModelConfig:
    """Read ``folder/config.json`` and return the typed config its architecture names."""
    return config_from_dict(read_config_json(folder))


_builtin_done = False


def _register_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from ..weights.llama import llama_checkpoint_map
    from .llama import LlamaConfig

    if "LlamaForCausalLM" not in _ARCHITECTURES:
        register_architecture("LlamaForCausalLM", LlamaConfig, llama_checkpoint_map)
