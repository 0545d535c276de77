"""The one registry from an architecture's name to its model.

``config.json`` carries ``architectures: ["Qwen3ForCausalLM"]``.  The name is
looked up here and gives the typed configuration class of that architecture;
the configuration turns itself into a :class:`ModelSpec`.  The reference has
no registry (tinyvllm/models/__init__.py:1-11 only re-exports its one model,
tinyvllm/bootstrap.py:70 imports it directly).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Protocol

from .spec import ModelSpec


class ConfigError(ValueError):
    """config.json is missing, malformed, or asks for what is not built."""


class ArchitectureConfig(Protocol):
    """What a typed architecture configuration has to offer."""

    @classmethod
    def from_json(cls, data: Mapping[str, Any]) -> "ArchitectureConfig": ...

    def to_json(self) -> dict[str, Any]: ...

    def to_spec(self) -> ModelSpec: ...


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type) -> None:
    """Make ``name`` (as written in config.json's ``architectures``) known."""
    for method in ("from_json", "to_json", "to_spec"):
        if not callable(getattr(config_class, method, None)):
            raise TypeError(f"{config_class.__name__} lacks {method}()")
    _ARCHITECTURES[name] = Architecture(name, config_class)


def architecture_names() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def lookup_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(architecture_names()) or "none"
        raise ConfigError(f"unknown architecture {name!r}; registered: {known}") from None


def parse_model_config(data: Any):
    """Typed configuration of a parsed config.json."""
    if not isinstance(data, Mapping):
        raise ConfigError("config.json must hold a JSON object")
    names = data.get("architectures")
    if not isinstance(names, list) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError("config.json must name exactly one entry in 'architectures'")
    return lookup_architecture(names[0]).config_class.from_json(data)


def read_model_config(model_dir: str | Path):
    """Typed configuration of the model folder ``model_dir``."""
    path = Path(model_dir) / "config.json"
    try:
        data = json.loads(path.read_text(encoding="utf-8"))
    except OSError as exc:
        raise ConfigError(f"cannot read {path}: {exc}") from exc
    except (UnicodeError, json.JSONDecodeError) as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    return parse_model_config(data)
