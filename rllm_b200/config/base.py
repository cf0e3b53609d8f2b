"""Typed model configuration and the one registry from architecture name to model.

A `config.json` names its architecture (`architectures[0]`, else `model_type`);
the registry maps that name to a typed configuration class and to the function
that builds the model from it. Parity: the reference's serde `ModelConfig`
(src/model/config.rs:332-612), `ModelArch::from_model_type`
(src/model/config.rs:300-320) and the `create_forward` match
(src/engine/loader.rs:163-205), folded into one table here.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of every typed configuration. Subclasses add the architecture's keys
    and implement `from_dict` / `to_dict` with the architecture's own key names."""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:  # pragma: no cover - abstract
        raise NotImplementedError


@dataclass(frozen=True)
class Architecture:
    name: str                      # e.g. "LlamaForCausalLM"
    model_types: tuple[str, ...]   # e.g. ("llama",)
    config_cls: type
    build: Callable[[Any], Any]    # typed config -> models.Model (no weights yet)


_REGISTRY: dict[str, Architecture] = {}
_BY_MODEL_TYPE: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build: Callable[[Any], Any],
                          model_types: tuple[str, ...] = ()) -> Architecture:
    """Add an architecture. This call, with new parts where the architecture
    needs them, is all that a new model family takes."""
    arch = Architecture(name, tuple(model_types), config_cls, build)
    _REGISTRY[name] = arch
    for mt in model_types:
        _BY_MODEL_TYPE[mt] = arch
    return arch


def registered_architectures() -> list[str]:
    return sorted(_REGISTRY)


def resolve_architecture(raw: dict[str, Any]) -> Architecture:
    names = raw.get("architectures") or []
    for n in names:
        if n in _REGISTRY:
            return _REGISTRY[n]
    mt = raw.get("model_type")
    if mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    raise ConfigError(
        f"unsupported architecture: architectures={names!r}, model_type={mt!r}; "
        f"registered: {registered_architectures()} "
        f"(model types {sorted(_BY_MODEL_TYPE)})")


def config_from_dict(raw: dict[str, Any]) -> tuple[Architecture, ModelConfig]:
    if "text_config" in raw and isinstance(raw["text_config"], dict):
        # multimodal wrappers keep the decoder's keys one level down
        # (src/model/config.rs:777-1035 unwraps the same way)
        inner = dict(raw["text_config"])
        inner.setdefault("architectures", raw.get("architectures"))
        raw = inner
    arch = resolve_architecture(raw)
    return arch, arch.config_cls.from_dict(raw)


def load_config(model_dir: str) -> tuple[Architecture, ModelConfig]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    with open(path) as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    # special token ids may stand in generation_config.json instead (checkpoints of the Llama 3
    # family keep the list of end tokens there)
    gen = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen):
        try:
            with open(gen) as f:
                extra = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{gen}: not valid JSON ({e})") from e
        if isinstance(extra, dict):
            for key in ("bos_token_id", "eos_token_id"):
                if raw.get(key) is None and extra.get(key) is not None:
                    raw[key] = extra[key]
    return config_from_dict(raw)


def require_int(raw: dict, key: str, *, minimum: int = 1, default: int | None = None) -> int:
    v = raw.get(key, default)
    if v is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config key {key!r} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config key {key!r} must be >= {minimum}, got {v}")
    return v


def require_float(raw: dict, key: str, *, default: float | None = None,
                  aliases: tuple[str, ...] = ()) -> float:
    v = raw.get(key)
    for a in aliases:
        if v is None:
            v = raw.get(a)
    if v is None:
        v = default
    if v is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config key {key!r} must be a number, got {v!r}")
    return float(v)
