"""The one registry from an architecture's name to its model.

An entry holds the function that turns config.json into a ``ModelSpec`` and
the function that builds the model from that spec.  ``architectures[0]`` of
config.json selects the entry, as the reference selects its executor from
config.json alone (src/model/spec.rs:138-168).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional

from ..errors import ConfigError, Unsupported
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    read_spec: Callable[[dict], ModelSpec]
    build_model: Callable      # (spec, ModelContext, source) -> model object with the DecoderModel interface
    adapt_source: Optional[Callable] = None   # (weight source) -> weight source under the names the spec uses

    def source_for(self, source):
        return self.adapt_source(source) if self.adapt_source is not None else source


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, read_spec, build_model, adapt_source=None) -> Architecture:
    """adapt_source: for checkpoints of the architecture that store the same tensors under other names."""
    arch = Architecture(name, read_spec, build_model, adapt_source)
    ARCHITECTURES[name] = arch
    return arch


def architecture_of(config: dict) -> Architecture:
    names = config.get("architectures")
    if not isinstance(names, list) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError("config.json: 'architectures' must be a list holding exactly one name")
    if names[0] not in ARCHITECTURES:
        raise Unsupported(f"architecture {names[0]!r} is not registered "
                          f"(registered: {sorted(ARCHITECTURES)})")
    return ARCHITECTURES[names[0]]


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    if os.path.getsize(path) > 64 << 20:       # src/artifact/mod.rs:603-619
        raise ConfigError(f"{path}: config.json exceeds 64 MiB")
    with open(path) as f:
        try:
            config = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: {e}") from None
    if not isinstance(config, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config


def spec_from_config(config: dict) -> ModelSpec:
    return architecture_of(config).read_spec(config)
