"""One registry from an architecture's name (``config.json["architectures"][0]``) to how it is built.

The reference hard-wires its model class (oxr_runtime/engine.py:214); here the name in config.json picks an
:class:`Architecture`: how to type the config and how to turn it into a :class:`ModelSpec` (a description
made only of registered parts). Adding an architecture = one ``register_architecture`` call; nothing in the
loader, cache, step function, scheduler or replay program names a model.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any], Mapping[str, Any] | None], Any]
    """(config.json, generation_config.json or None) -> typed config."""
    model_spec: Callable[[Any], Any]
    """typed config -> :class:`oxr_inference_b200.parts.spec.ModelSpec`."""


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    if arch.name in ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    ARCHITECTURES[arch.name] = arch
    return arch


def _load_builtin() -> None:
    # Imported for its side effect: each module under ``models`` registers itself.
    import oxr_inference_b200.models  # noqa: F401


def resolve_architecture(raw_config: Mapping[str, Any]) -> Architecture:
    from oxr_inference_b200.config.model_config import ConfigError

    _load_builtin()
    names = raw_config.get("architectures")
    if not names:
        raise ConfigError(f"config.json has no 'architectures' entry; known: {sorted(ARCHITECTURES)}")
    name = names[0]
    if name not in ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; known: {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[name]
