"""One registry from an architecture's name (config.json `architectures[0]`)
to its typed configuration and to the function that lays the model out.

The reference has no registry: it sniffs substrings of `general.architecture`
into booleans (picolm/model_gguf.c:729-751) and treats the plain transformer as
the default branch.  Here an unknown name is an error that lists what is known.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, build_spec) -> None:
    """Make `name` loadable.  `config_from_dict(raw)` returns the typed
    configuration; `build_spec(config)` returns the `ModelSpec`."""
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise KeyError(
            "config.json lacks the key 'architectures'; registered: " + ", ".join(registered_architectures()))
    name = str(archs[0])
    if name not in _ARCHITECTURES:
        raise KeyError(
            f"architecture {name!r} is not registered; registered: " + ", ".join(registered_architectures()))
    return _ARCHITECTURES[name]


def read_config(model_dir_or_json: str):
    """Read a model folder's config.json (or a config.json path) into the typed
    configuration of its architecture."""
    path = model_dir_or_json
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    return config_from_dict(raw)


def config_from_dict(raw: Mapping[str, Any]):
    return architecture_of(raw).config_from_dict(raw)


def spec_of(config) -> ModelSpec:
    """The model layout of a typed configuration, through the registry."""
    name = getattr(config, "architecture", None)
    if name not in _ARCHITECTURES:
        raise KeyError(
            f"architecture {name!r} is not registered; registered: " + ", ".join(registered_architectures()))
    spec = _ARCHITECTURES[name].build_spec(config)
    spec.validate()
    return spec
