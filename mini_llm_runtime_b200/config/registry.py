"""Registries: architecture name -> (config class, plan builder); part kind -> class.

One table per kind of thing.  An architecture is added with
`register_architecture`, a part with `register_part`; nothing else in the package
names a concrete architecture or part, so either can be added from outside the
package (a test registers a toy mixer this way).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Tuple, Type

from .base import ConfigError, ModelPlan

PART_KINDS = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "lm_head")

_architectures: Dict[str, Tuple[type, Callable[[object], ModelPlan]]] = {}
_parts: Dict[str, Dict[str, type]] = {k: {} for k in PART_KINDS}


def register_architecture(name: str, config_cls: type, plan_builder: Callable[[object], ModelPlan]) -> None:
    """`config_cls.from_dict(dict)` parses config.json; `plan_builder(config)` gives the plan."""
    _architectures[name] = (config_cls, plan_builder)


def known_architectures():
    return sorted(_architectures)


def architecture(name: str):
    try:
        return _architectures[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; known: {known_architectures()}") from None


def register_part(category: str, kind: str, cls: type) -> None:
    if category not in _parts:
        raise KeyError(f"part category {category!r} is not one of {PART_KINDS}")
    _parts[category][kind] = cls


def part_class(category: str, kind: str) -> type:
    try:
        return _parts[category][kind]
    except KeyError:
        raise ConfigError(f"unknown {category} kind {kind!r}; known: {sorted(_parts.get(category, {}))}") from None


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path} not found") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None


def config_from_dict(raw: dict):
    """Pick the config class by `architectures[0]` and parse."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"config.json needs a non-empty 'architectures' list; known: {known_architectures()}")
    config_cls, _ = architecture(archs[0])
    return config_cls.from_dict(raw)


def config_from_dir(model_dir: str):
    return config_from_dict(read_config_json(model_dir))


def plan_for(config) -> ModelPlan:
    _, builder = architecture(config.architecture)
    plan = builder(config)
    plan.validate()
    return plan
