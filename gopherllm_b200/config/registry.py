"""One registry from an architecture's declared name to its definition.

The reference resolves a declared label through an alias table and generic
spelling rules (arch_detect.go:58-110: lower-case, ``-``/``_`` variants,
Hugging Face class-name suffixes stripped) and rejects what is left with
"unsupported architecture: %s" (runtime.go:533).  The same rules apply here to
``architectures[0]`` and ``model_type`` of a config.json.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

_CLASS_SUFFIXES = ("forcausallm", "forconditionalgeneration",
                   "forsequenceclassification", "lmheadmodel", "model")


@dataclass(frozen=True)
class Architecture:
    """What the framework needs to know about one architecture.

    name: canonical label.
    config_class: typed configuration with ``from_dict(dict)`` and ``to_dict()``.
    build_spec: config -> ModelSpec (layers, schedule, sizes).
    tensor_names: config -> TensorNames (part parameter -> tensor name in the file).
    """
    name: str
    config_class: type
    build_spec: Callable
    tensor_names: Callable


_ARCHITECTURES: Dict[str, Architecture] = {}
_ALIASES: Dict[str, str] = {}


def _squash(label: str) -> str:
    return label.replace("-", "").replace("_", "")


def register_architecture(arch: Architecture, aliases: List[str] = ()) -> None:
    key = _squash(arch.name.lower())
    _ARCHITECTURES[key] = arch
    for a in aliases:
        _ALIASES[_squash(a.lower())] = key


def known_architectures() -> List[str]:
    return sorted({a.name for a in _ARCHITECTURES.values()} | set(_ALIASES))


def _lookup(label: str) -> Optional[Architecture]:
    key = _squash(label)
    if key in _ARCHITECTURES:
        return _ARCHITECTURES[key]
    if key in _ALIASES:
        return _ARCHITECTURES[_ALIASES[key]]
    return None


def resolve_architecture(label: str) -> Optional[Architecture]:
    """Canonical architecture for a declared label, or None."""
    lower = (label or "").strip().lower()
    if not lower:
        return None
    hit = _lookup(lower)
    if hit is not None:
        return hit
    for suffix in _CLASS_SUFFIXES:
        if lower.endswith(suffix) and len(lower) > len(suffix):
            hit = _lookup(lower[: -len(suffix)])
            if hit is not None:
                return hit
    return None


def architecture_from_config(cfg: dict) -> Architecture:
    """Pick the architecture a config.json declares: ``architectures[0]``
    first, then ``model_type``."""
    declared = []
    archs = cfg.get("architectures")
    if isinstance(archs, (list, tuple)):
        declared += [a for a in archs if isinstance(a, str)]
    if isinstance(cfg.get("model_type"), str):
        declared.append(cfg["model_type"])
    for label in declared:
        arch = resolve_architecture(label)
        if arch is not None:
            return arch
    shown = ", ".join(declared) if declared else "<none declared>"
    raise ValueError(f"unsupported architecture: {shown} (known: {', '.join(known_architectures())})")
