"""Architecture-neutral description of a model: which parts, with which sizes,
bound to which checkpoint tensors, run in which order.

An architecture (see ``gibbs_b200.config.registry``) turns its ``config.json``
into a ``ModelPlan``.  Everything below the plan (weight loader, parts, cache
manager, step function) reads the plan only and never asks which model it is
in.  Mixed models are expressed here: every layer names its own mixer and
feed-forward kind, and ``order`` is a list that may run a layer twice or let
an entry read the cache of an earlier entry.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: its registry ``kind``, its sizes and constants (``params``)
    and the checkpoint tensor behind each of its local tensor names."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    tensors: dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A block: the registry kind of its arrangement (``block``), the parts it
    is made of as (role, category, PartSpec) in the arrangement's own order,
    and the arrangement's constants.  Which roles there are is the
    arrangement's business: pre-norm residual has a norm before the mixer and
    one before the feed-forward; another may add norms after them, share one
    norm between two parallel branches, or have no feed-forward at all."""

    block: str
    parts: tuple[tuple[str, str, PartSpec], ...]
    params: dict[str, Any] = field(default_factory=dict)

    def part(self, role: str) -> PartSpec:
        for r, _, spec in self.parts:
            if r == role:
                return spec
        raise KeyError(f"the '{self.block}' layer has no part in the role '{role}'; it has "
                       f"{[r for r, _, _ in self.parts]}")

    def __getattr__(self, role: str) -> PartSpec:
        # layer.mixer, layer.ffn, ...: the part in that role
        if role.startswith("_") or role in ("block", "parts", "params"):
            raise AttributeError(role)
        try:
            return self.part(role)
        except KeyError as e:
            raise AttributeError(str(e)) from None


def prenorm_layer(mixer_norm: PartSpec, mixer: PartSpec, ffn_norm: PartSpec, ffn: PartSpec) -> LayerSpec:
    """The arrangement x += mixer(norm(x)); x += ffn(norm(x))."""
    return LayerSpec("prenorm_residual", (("mixer_norm", "norm", mixer_norm), ("mixer", "mixer", mixer),
                                          ("ffn_norm", "norm", ffn_norm), ("ffn", "feed_forward", ffn)))


@dataclass(frozen=True)
class OrderEntry:
    """One run of a layer.  Each entry owns a cache of its own unless
    ``reads_cache_of`` names an earlier entry (by its index in ``order``)
    whose cache this run only reads."""

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_context: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[OrderEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        for i, e in enumerate(self.order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {e.layer}; the plan has {len(self.layers)} layers")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < i:
                    raise ValueError(
                        f"order[{i}] reads the cache of entry {e.reads_cache_of}, which does not run before it")
                if self.order[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"order[{i}] reads the cache of entry {e.reads_cache_of}, which owns none")
