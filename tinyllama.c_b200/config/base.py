"""Typed model configurations read from config.json, and the architecture registry.

CodeClaper/tinyllama.c derives its ``ArchConfig`` from GGUF metadata with per-field
fallbacks (core.c:1563-1653) and picks the model by the architecture string
(core.c:473-489, 2037-2049).  Here the metadata is the architecture's own
``config.json``; every size and constant of a model is a field of a config class,
and one registry maps ``architectures[0]`` to (config class, model builder).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, Dict, Tuple


class ConfigError(ValueError):
    """config.json is missing a key, has a wrong type, or its sizes contradict each other."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses declare their config.json keys as dataclass fields (a field without a
    default is required), normalise and check them in ``validate`` and describe their
    layers in ``layer_specs``."""

    architecture: str

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        archs = raw.get("architectures")
        if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of strings")
        kwargs: Dict[str, Any] = {"architecture": archs[0]}
        problems = []
        for f in fields(cls):
            if f.name == "architecture":
                continue
            if f.name in raw and raw[f.name] is not None:
                kwargs[f.name] = raw[f.name]
            elif f.default is dataclass_missing and f.default_factory is dataclass_missing:
                problems.append(f"missing key '{f.name}'")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        try:
            cfg = cls(**kwargs)
        except TypeError as e:  # pragma: no cover - defensive
            raise ConfigError(f"config.json: {e}") from e
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architectures": [self.architecture]}
        for f in fields(self):
            if f.name != "architecture":
                v = getattr(self, f.name)
                out[f.name] = list(v) if isinstance(v, tuple) else v
        return out

    def validate(self) -> None:  # overridden
        pass


from dataclasses import MISSING as dataclass_missing  # noqa: E402  (used in from_dict)


# ---- registry ------------------------------------------------------------------------
_ARCHITECTURES: Dict[str, Tuple[type, Callable]] = {}


def register_architecture(name: str, config_cls: type, builder: Callable) -> None:
    """Registers ``name`` (the string in config.json's ``architectures``) with the class
    that parses its config and the function ``builder(config) -> Model`` that lays out
    its parts."""
    _ARCHITECTURES[name] = (config_cls, builder)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> Tuple[type, Callable]:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; registered: {registered_architectures()}")
    return _ARCHITECTURES[name]


def config_from_dict(raw: Dict[str, Any]) -> ModelConfig:
    archs = raw.get("architectures") if isinstance(raw, dict) else None
    if not (isinstance(archs, list) and archs):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of strings")
    config_cls, _ = lookup_architecture(archs[0])
    return config_cls.from_dict(raw)


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError as e:
        raise ConfigError(f"{path}: no such file") from e
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    return config_from_dict(raw)
