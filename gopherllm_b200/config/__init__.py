"""Typed configurations, architecture-neutral specs and the architecture registry."""
from __future__ import annotations

import json
import os

from .registry import (Architecture, architecture_from_config, known_architectures,
                       register_architecture, resolve_architecture)
from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec,
                    PositionSpec, ScheduleEntry, default_schedule)
from . import phi as _phi  # registers the architecture
from .phi import PhiConfig


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{folder}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def load_config(folder: str):
    """(architecture, typed config) for a model folder; the class is chosen by
    what config.json declares."""
    raw = read_config_json(folder)
    arch = architecture_from_config(raw)
    return arch, arch.config_class.from_dict(raw)
