"""Base class of typed model configurations and the helpers to read config.json."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Optional

from .layout import ModelLayout


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine cannot run."""


class ModelConfig:
    """What every architecture's configuration offers to the engine.

    Subclasses are dataclasses whose fields are the architecture's own
    config.json keys.  ``layout()`` is the only thing the engine builds from.
    """

    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def layout(self) -> ModelLayout:
        raise NotImplementedError

    # Tokens that end a request, from config.json (eos_token_id may be a list).
    def stop_token_ids(self) -> tuple[int, ...]:
        return ()

    def max_positions(self) -> int:
        raise NotImplementedError


@dataclass
class GenerationDefaults:
    """Sampling defaults in the reference's names (mstar/utils/sampling.py:207-226,
    mstar/model/orpheus/config.py:44-48), read from generation_config.json if the
    model folder has one."""

    temperature: float = 0.6
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    ignore_eos: bool = False
    max_new_tokens: int = 2048
    extra: dict = field(default_factory=dict)

    @classmethod
    def from_folder(cls, folder: str | Path) -> "GenerationDefaults":
        path = Path(folder) / "generation_config.json"
        out = cls()
        if not path.is_file():
            return out
        raw = json.loads(path.read_text())
        for key in ("temperature", "top_k", "top_p", "repetition_penalty", "ignore_eos",
                    "max_new_tokens"):
            if key in raw and raw[key] is not None:
                setattr(out, key, type(getattr(out, key))(raw[key]))
        return out


def read_config_json(folder: str | Path) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and "
                                "model.safetensors")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc


def require(raw: Mapping[str, Any], key: str, kind: type, missing: list[str]) -> Any:
    """Fetch a required key, recording it in ``missing`` rather than raising so
    that one error can list every absent key."""
    if key not in raw or raw[key] is None:
        missing.append(key)
        return kind()
    return _coerce(key, raw[key], kind)


def optional(raw: Mapping[str, Any], key: str, kind: type, default: Optional[Any]) -> Any:
    if key not in raw or raw[key] is None:
        return default
    return _coerce(key, raw[key], kind)


def _coerce(key: str, value: Any, kind: type) -> Any:
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config key {key!r} must be true or false, got {value!r}")
        return value
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise ConfigError(f"config key {key!r} must be an integer, got {value!r}")
        return int(value)
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config key {key!r} must be a number, got {value!r}")
        return float(value)
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config key {key!r} must be a string, got {value!r}")
        return value
    return value
