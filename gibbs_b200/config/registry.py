"""One registry from an architecture's name to the code that reads its
config.json and lays out its plan.

MisterTK/gibbs picks a family by ``architectures`` / ``model_type``
(``src/arch/mod.rs:723-759``; LFM2's match rule: ``arch/families/lfm2.json5:6``).
Here an architecture registers a function ``(config dict, tensor names or None)
-> typed configuration`` whose ``plan()`` returns a ``ModelPlan``; nothing else
in the framework names an architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterable, Optional


@dataclass(frozen=True)
class Architecture:
    name: str
    model_types: tuple[str, ...]
    parse: Callable[[dict, Optional[Iterable[str]]], object]   # -> typed config with .plan()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse, model_types: Iterable[str] = ()) -> None:
    _ARCHITECTURES[name] = Architecture(name, tuple(model_types), parse)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def detect(cfg: dict, forced: Optional[str] = None) -> Architecture:
    """The architecture a config.json names: by ``architectures`` first, then
    by ``model_type``; ``forced`` skips detection (the reference's ``--arch``,
    ``src/main.rs:180-183``)."""
    if forced is not None:
        if forced in _ARCHITECTURES:
            return _ARCHITECTURES[forced]
        for a in _ARCHITECTURES.values():
            if forced in a.model_types:
                return a
        raise KeyError(f"unknown architecture '{forced}'; known: {known_architectures()}")
    for name in cfg.get("architectures") or []:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    mt = cfg.get("model_type")
    for a in _ARCHITECTURES.values():
        if mt is not None and mt in a.model_types:
            return a
    raise KeyError(
        f"config.json names architectures {cfg.get('architectures')} / model_type {mt!r}; "
        f"known: {known_architectures()}")


def parse_config(cfg: dict, tensor_names=None, forced: Optional[str] = None):
    return detect(cfg, forced).parse(cfg, tensor_names)
