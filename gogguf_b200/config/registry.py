"""Architecture registry: architecture name -> typed configuration class.

The reference dispatches on ``general.architecture`` with a switch and fails
on unknown names (pkg/model/model.go:23-48).  Here the dispatch is a table so
that an architecture is added by one `register_architecture` call; the key is
``architectures[0]`` of config.json, with ``model_type`` as an alias.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Type

_ARCHITECTURES: Dict[str, Type] = {}


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, bad value, unknown architecture."""


def register_architecture(*names: str) -> Callable[[Type], Type]:
    """Class decorator: make a config class reachable under the given names.

    The class must provide ``from_dict(d) -> config`` and the instance
    ``to_spec() -> ModelSpec``, ``to_dict() -> dict`` (its config.json).
    """

    def deco(cls: Type) -> Type:
        for n in names:
            if n in _ARCHITECTURES and _ARCHITECTURES[n] is not cls:
                raise ValueError(f"architecture {n!r} is already registered")
            _ARCHITECTURES[n] = cls
        return cls

    return deco


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(cfg: Dict[str, Any]) -> str:
    archs = cfg.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return str(archs[0])
    if "model_type" in cfg:
        return str(cfg["model_type"])
    raise ConfigError("config.json names no architecture (neither 'architectures' nor 'model_type')")


def config_class_for(name: str) -> Type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"architecture {name!r} is not supported; registered: {registered_architectures()}"
        ) from None


def config_from_dict(cfg: Dict[str, Any]):
    """Typed configuration for a parsed config.json."""
    name = architecture_name(cfg)
    try:
        cls = config_class_for(name)
    except ConfigError:
        # `architectures[0]` unknown: fall back to model_type before giving up.
        mt = cfg.get("model_type")
        if mt is None or mt not in _ARCHITECTURES:
            raise
        cls = _ARCHITECTURES[mt]
    return cls.from_dict(cfg)


def load_config(path: str):
    """Read ``config.json`` from a model folder (or a path to the json itself)."""
    p = os.path.join(path, "config.json") if os.path.isdir(path) else path
    if not os.path.isfile(p):
        raise ConfigError(f"no config.json at {p}")
    with open(p, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{p}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{p}: top level must be an object")
    _merge_generation_config(d, os.path.join(os.path.dirname(p), "generation_config.json"))
    return config_from_dict(d)


def _merge_generation_config(d: Dict[str, Any], path: str) -> None:
    """A model folder may name further end-of-sequence ids in ``generation_config.json`` (a chat
    model's end-of-turn id beside its end-of-text id); generation stops on any of them, the ones of
    config.json first.  An unreadable file is an error, a missing one is not."""
    if not os.path.isfile(path):
        return
    with open(path, "r", encoding="utf-8") as f:
        try:
            g = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    extra = g.get("eos_token_id") if isinstance(g, dict) else None
    if extra is None:
        return
    def ids(v):
        return [int(x) for x in v] if isinstance(v, (list, tuple)) else ([] if v is None else [int(v)])
    merged = ids(d.get("eos_token_id"))
    for t in ids(extra):
        if t not in merged:
            merged.append(t)
    d["eos_token_id"] = merged if len(merged) != 1 else merged[0]
