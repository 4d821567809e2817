"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

The reference whitelists by ``config.model_type`` (utils/architecture.py:16,53-54) and inspects
a Hugging Face module tree; this engine keys on the architecture name and builds everything
from config.json alone.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict

from .errors import UnsupportedModelError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type                      # has from_dict(dict) and to_dict()
    build_spec: Callable[[object], ModelSpec]  # typed config -> ModelSpec


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable[[object], ModelSpec]) -> Architecture:
    architecture = Architecture(name, config_class, build_spec)
    ARCHITECTURES[name] = architecture
    return architecture


def architecture_of(raw_config: dict) -> Architecture:
    names = raw_config.get("architectures") or []
    if not names:
        raise UnsupportedModelError("config.json has no 'architectures' entry; cannot choose a model")
    if names[0] not in ARCHITECTURES:
        raise UnsupportedModelError(
            f"Architecture {names[0]!r} is not supported (supported: {', '.join(sorted(ARCHITECTURES))})")
    return ARCHITECTURES[names[0]]


def read_config(model_dir: str):
    """(typed config, Architecture) of the model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir!r} has no config.json")
    with open(path) as handle:
        raw = json.load(handle)
    architecture = architecture_of(raw)
    return architecture.config_class.from_dict(raw), architecture
