"""Interfaces of the parts a model is put together from, and the registries
that map a plan's ``kind`` strings to their classes.

A part
  * declares the tensors it needs (``declare(params)``: local name ->
    ``TensorDecl``), so that the loader can check a checkpoint before anything
    is copied;
  * is built from ``(params, tensors, runtime)``, where ``tensors`` maps its
    local names to device tensors already in their in-memory dtype;
  * knows its own sizes only: nothing tells it which model, layer index or
    architecture it belongs to.

Categories and what each must implement:

  norm        ``forward(x, out=None, rows=None) -> [N or len(rows), dim]`` in the
              compute dtype; x is the ``Residual`` stream (or a float32 tensor).
  position    ``rotary() -> Rotary | None`` (tables a mixer's kernel applies)
              and ``embed(x_f32, step)`` (an in-place hook on the embedded
              tokens; default nothing).
  mixer       ``cache_needs() -> [PagedKV | SlotState, ...]`` and
              ``forward(h, residual, step, caches)`` which ADDS the mixer's
              output into the ``Residual`` stream (``residual.add_(y)``, or a
              projection called with ``out=residual, accumulate=True``);
              ``caches`` holds one view per need.
  feed_forward ``forward(h, residual, step)``, adding likewise.
  block       an arrangement of parts around the residual stream.  Its class
              names the roles it is made of (``ROLES``: (role, category) pairs);
              a plan's layer gives one part per role; the block is built from
              ``{role: part}`` and implements ``forward(residual, step, caches)``.
              ``caches`` holds the views of all its parts' cache needs, in the
              order of the roles (``caches_of(role, caches)`` picks a part's).
  Optionally every part has ``plan_ops(plan, ...)`` with the arguments of its
  ``forward`` minus the step and the residual: it appends the same work as
  operations of a step plan (``engine/plan.py``), which the engine then runs
  with one call per step instead of one per kernel.
  embedding   ``forward(ids_i32 [N]) -> x_f32 [N, dim]``.
  head        ``forward(z [R, dim]) -> logits_f32 [R, vocab]``.

The residual stream is 32-bit in every compute dtype, so the residual sum is
exact to 32-bit rounding.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import torch

# roles decide the dtype a checkpoint tensor gets in memory (see weights.loader)
MATRIX = "matrix"     # operand of a matrix product, or an embedding table
VECTOR = "vector"     # gains, biases, filter taps: always 32-bit in memory
INT_TABLE = "int"     # integer tables: int32 in memory


@dataclass(frozen=True)
class TensorDecl:
    shapes: tuple[tuple[int, ...], ...]   # accepted checkpoint shapes; the first is what the part receives
    role: str = MATRIX

    @staticmethod
    def of(*shape: int, role: str = MATRIX) -> "TensorDecl":
        return TensorDecl((tuple(shape),), role)


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position (or of the last ``window`` positions)
    in pages: keys [n_pages, kv_heads, page_size, head_dim], values
    [n_pages, kv_heads, page_size, v_head_dim] (``v_head_dim`` None: as the keys)."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class SlotState:
    """Per-request state of fixed size, zero when a request starts."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What a part needs to know about where and how it computes."""
    dtype: torch.dtype                 # compute dtype: torch.float32 or torch.bfloat16
    device: torch.device

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)


class Residual:
    """The 32-bit residual stream of a step, [tokens, hidden], plus at most one
    set of partial sums that a split-K product left to be added to it.  The
    next norm adds them while it reads the stream (one kernel instead of
    three); anything else that needs the values calls ``tensor()``."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending = None            # (partials [splits, tokens, hidden], bias or None)
        self.ssq = None                # partial sums of squares of the rows as they stand [parts, tokens], or None

    def tensor(self) -> torch.Tensor:
        """The stream with everything added (the caller may change it: what was known
        about its rows' sums of squares is dropped)."""
        self.ssq = None
        if self.pending is not None:
            from .. import ops
            ops.add_pending(self.x, *self.pending)
            self.pending = None
        return self.x

    def defer(self, partials: torch.Tensor, bias) -> None:
        self.tensor()
        self.pending = (partials, bias)

    def take_pending(self):
        p, self.pending = self.pending, None
        return p

    def add_(self, y: torch.Tensor) -> "Residual":
        """For parts written with tensor operations: stream += y."""
        self.tensor().add_(y.to(torch.float32))
        return self

    @property
    def shape(self):
        return self.x.shape


class NotPlannable(Exception):
    """Raised while a step plan is built when a part (or one of its sizes)
    cannot be written as operations of the plan; the engine then runs the
    parts' ``forward`` methods from Python."""


def plan_ops_of(part):
    """``part.plan_ops``, or NotPlannable for a part that has none (parts need
    not derive from the classes below)."""
    fn = getattr(part, "plan_ops", None)
    if fn is None:
        raise NotPlannable(f"{type(part).__name__} has no plan operations")
    return fn


class Part:
    category: str = ""

    @classmethod
    def declare(cls, params: dict) -> dict[str, TensorDecl]:
        return {}

    def __init__(self, params: dict, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.params, self.rt = params, rt

    def kernel_libraries(self) -> Sequence[str]:
        """Kernel libraries this part launches from (built before the first step)."""
        return ("core",)

    def plan_ops(self, plan, *args):
        """Append to ``plan`` (an ``engine.plan.PlanBuilder``) the operations
        that do what ``forward`` does, for any step.  Optional: a model with a
        part that lacks it is run through the ``forward`` methods."""
        raise NotPlannable(f"{type(self).__name__} has no plan operations")


class Norm(Part):
    category = "norm"

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def lazy(self, x, rows: Optional[torch.Tensor] = None):
        """For a consumer that says ``fuses_norm``: the normalised rows, or an object that
        a product can read *through* the norm (``ops.NormedRows``), so that no kernel runs
        for the norm alone.  By default the norm simply runs."""
        return self.forward(x, rows=rows)


@dataclass(frozen=True)
class Rotary:
    inv_freq: torch.Tensor    # float32 [rotary_dim / 2]
    rotary_dim: int
    adjacent_pairs: bool      # pairs (2j, 2j+1) instead of (j, j + rotary_dim/2)
    mscale: float = 1.0       # the cosines and sines are multiplied by this

    def __post_init__(self):
        # what the kernels read: the frequencies followed by the factor
        tail = torch.tensor([self.mscale], dtype=torch.float32, device=self.inv_freq.device)
        object.__setattr__(self, "table", torch.cat([self.inv_freq.to(torch.float32).reshape(-1), tail]).contiguous())


class PositionEncoding(Part):
    category = "position"

    def rotary(self) -> Optional[Rotary]:
        return None

    def embed(self, x: torch.Tensor, step) -> None:
        return None


class Mixer(Part):
    category = "mixer"
    # False for a mixer whose forward reads the step's host-side lists or otherwise cannot be
    # recorded into a CUDA graph; the engine then runs decode steps without graphs.
    capturable = True

    def cache_needs(self) -> list:
        return []

    def forward(self, h: torch.Tensor, residual: torch.Tensor, step, caches: list) -> None:
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, h: torch.Tensor, residual: torch.Tensor, step) -> None:
        raise NotImplementedError


def tensor_bytes(obj, seen: set) -> int:
    """Bytes of the floating-point tensors an object (and the helpers it
    holds) keeps, each tensor counted once across calls that share ``seen``."""
    total = 0
    if id(obj) in seen:
        return 0
    seen.add(id(obj))
    values = obj.values() if isinstance(obj, dict) else vars(obj).values() if hasattr(obj, "__dict__") else ()
    for v in values:
        if isinstance(v, torch.Tensor):
            if v.is_floating_point() and v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                total += v.numel() * v.element_size()
        elif isinstance(v, (list, tuple)):
            total += sum(tensor_bytes(u, seen) for u in v if hasattr(u, "__dict__") or isinstance(u, dict))
        elif (hasattr(v, "__dict__") or isinstance(v, dict)) and not isinstance(v, (Runtime, type)):
            total += tensor_bytes(v, seen)
    return total


def step_weight_bytes(part, n_tokens: int, seen: set) -> int:
    """Bytes of weights ``part`` reads in a step of ``n_tokens`` tokens when
    each is read once.  A part whose step reads only some of its weights (a
    feed-forward that routes among experts) says so with a method
    ``step_weight_bytes(n_tokens, seen)`` of its own; for every other part it
    is all its floating-point tensors."""
    own = getattr(part, "step_weight_bytes", None)
    if own is not None:
        return int(own(n_tokens, seen))
    return tensor_bytes(part, seen)


class Block:
    """An arrangement of parts around the residual stream.  ``ROLES`` names
    what it is made of; ``build_model`` checks a plan's layer against it and
    hands the parts over as ``{role: part}`` (also reachable as attributes)."""
    category = "block"
    ROLES: tuple = ()

    def __init__(self, parts: dict, rt: Runtime, params: Optional[dict] = None):
        self.parts, self.rt, self.params = dict(parts), rt, dict(params or {})
        for role, part in self.parts.items():
            setattr(self, role, part)
        self._cache_slices: dict = {}
        at = 0
        for role, part in self.parts.items():
            needs = getattr(part, "cache_needs", None)
            n = len(needs()) if needs is not None else 0
            self._cache_slices[role] = (at, at + n)
            at += n

    def cache_needs(self) -> list:
        """The cache needs of all parts of the block, in the order of its roles."""
        out = []
        for part in self.parts.values():
            needs = getattr(part, "cache_needs", None)
            if needs is not None:
                out += list(needs())
        return out

    def caches_of(self, role: str, caches: list) -> list:
        """The views that belong to the part in ``role``.  A block with one part that keeps
        a cache hands it everything it was given (an entry that reads another entry's cache
        gets that entry's views, whatever its own needs are)."""
        holders = [r for r, p in self.parts.items() if getattr(p, "cache_needs", None) is not None]
        if holders == [role]:
            return caches
        lo, hi = self._cache_slices[role]
        return caches[lo:hi]

    @property
    def capturable(self) -> bool:
        """Whether a decode step through this block can be recorded into a CUDA graph."""
        return all(getattr(p, "capturable", True) for p in self.parts.values())

    def forward(self, x: torch.Tensor, step, caches: list) -> None:
        raise NotImplementedError

    def plan_ops(self, plan, caches: list) -> None:
        raise NotPlannable(f"{type(self).__name__} has no plan operations")


# ---------------------------------------------------------------------------
_REGISTRY: dict[tuple[str, str], Any] = {}
CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")


def register_part(category: str, kind: str, cls) -> None:
    """Make ``kind`` available to plans.  Registering a kind again replaces it."""
    if category not in CATEGORIES:
        raise KeyError(f"unknown part category '{category}'; known: {CATEGORIES}")
    _REGISTRY[(category, kind)] = cls


def part_class(category: str, kind: str):
    try:
        return _REGISTRY[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise KeyError(f"no {category} of kind '{kind}' is registered; known: {known}") from None
