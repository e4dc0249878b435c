"""Registries: architecture name -> (configuration class, builder), and part kind -> class.

An architecture is registered once with the class that parses its config.json and a
builder that turns that configuration into a ``ModelSpec`` (a declarative list of parts
with their parameters, their tensor names in the checkpoint, and the order in which the
layers run).  Parts (mixer, feed-forward, norm, position encoding, block arrangement)
are registered by a short kind name; a ``PartSpec`` refers to that name.  Tests register
toy parts and toy architectures through the same calls without touching this package.

The reference has no registry: it branches on attributes of the model object
(puneethgv/DiSpec dispec/engine/model_runner.py:74-84).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


class RegistryError(KeyError):
    def __str__(self) -> str:  # KeyError quotes its message; keep it readable
        return self.args[0] if self.args else ""


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_class: type
    builder: Callable  # (config) -> ModelSpec


_ARCHITECTURES: dict[str, ArchitectureEntry] = {}
_PARTS: dict[str, dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "block": {},
    "embedding": {}, "head": {},
}


def register_architecture(name: str, config_class: type, builder: Callable) -> None:
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_class, builder)


def architecture_entry(name: str) -> ArchitectureEntry:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise RegistryError(f"architecture {name!r} is not registered; known: "
                            f"{', '.join(sorted(_ARCHITECTURES)) or '(none)'}")
    return _ARCHITECTURES[name]


def architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def register_part(role: str, kind: str):
    """Class decorator: ``@register_part("mixer", "gqa_attention")``."""
    if role not in _PARTS:
        raise RegistryError(f"unknown part role {role!r}; roles: {', '.join(_PARTS)}")

    def deco(cls):
        _PARTS[role][kind] = cls
        cls.role, cls.kind = role, kind
        return cls

    return deco


def part_class(role: str, kind: str) -> type:
    _ensure_builtin()
    table = _PARTS.get(role)
    if table is None:
        raise RegistryError(f"unknown part role {role!r}; roles: {', '.join(_PARTS)}")
    if kind not in table:
        raise RegistryError(f"no {role} of kind {kind!r} is registered; known: "
                            f"{', '.join(sorted(table)) or '(none)'}")
    return table[kind]


_builtin_loaded = False


def _ensure_builtin() -> None:
    """Import the built-in parts and architectures on first use (they register themselves)."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    import dispec_b200.parts  # noqa: F401
    import dispec_b200.models  # noqa: F401
