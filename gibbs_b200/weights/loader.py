"""Binds checkpoint tensors to the parts of a plan by tensor name.

Before anything is copied, every tensor the plan's parts declare is compared
with what the checkpoint holds; all problems are reported in ONE error:
tensors that are missing, tensors no part reads (MisterTK/gibbs refuses
those too, ``src/runtime/lm.rs:357-367``) and tensors of the wrong shape.

In memory (``memory_dtype``): matrices stored in bfloat16 stay bfloat16 when
the model computes in bfloat16; a tensor stored in 32-bit stays 32-bit; gains,
biases and filter taps are always widened to 32-bit (exact); integer tables
become int32; with a float32 compute dtype everything is widened to 32-bit,
which makes the 32-bit run of a bfloat16 checkpoint its exact twin.
"""
from __future__ import annotations

from collections import Counter

import torch

from ..config.plan import ModelPlan, PartSpec
from ..parts.base import INT_TABLE, MATRIX, VECTOR, Runtime, TensorDecl, part_class


class WeightError(ValueError):
    """A checkpoint that does not fit its plan.  ``missing``, ``unexpected``
    and ``wrong_shape`` list every offending tensor."""

    def __init__(self, missing, unexpected, wrong_shape):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = ["the checkpoint does not match the model's configuration:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}):")
            lines += [f"    {n}  expected shape {list(s)}" for n, s in missing]
        if unexpected:
            lines.append(f"  unexpected tensors, read by no part ({len(unexpected)}):")
            lines += [f"    {n}  shape {list(s)}" for n, s in unexpected]
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}):")
            lines += [f"    {n}  expected {' or '.join(str(list(s)) for s in want)}, found {list(got)}"
                      for n, want, got in wrong_shape]
        super().__init__("\n".join(lines))


def memory_dtype(stored: torch.dtype, role: str, compute: torch.dtype) -> torch.dtype:
    if role == INT_TABLE:
        return torch.int32
    if role == VECTOR or compute == torch.float32:
        return torch.float32
    if stored == torch.bfloat16:
        return torch.bfloat16
    return torch.float32          # stored in 32-bit (or float16/64): kept / widened to 32-bit


class WeightBinder:
    def __init__(self, plan: ModelPlan, source, rt: Runtime):
        from ..parts.model import plan_parts
        self.plan, self.source, self.rt = plan, source, rt
        self.decls: dict[str, TensorDecl] = {}       # checkpoint name -> declaration
        self.uses: Counter = Counter()
        self._conflicts = []
        for category, spec in plan_parts(plan):
            for local, decl in part_class(category, spec.kind).declare(spec.params).items():
                if local not in spec.tensors:
                    raise KeyError(f"the plan binds no checkpoint tensor to '{local}' of the {spec.kind} part")
                name = spec.tensors[local]
                prev = self.decls.get(name)
                if prev is not None and prev.shapes[0] != decl.shapes[0]:
                    self._conflicts.append((name, prev.shapes, decl.shapes[0]))
                self.decls.setdefault(name, decl)
                self.uses[name] += 1
        self._shared: dict[str, torch.Tensor] = {}

    def verify(self) -> None:
        have = set(self.source.names())
        missing = [(n, d.shapes[0]) for n, d in self.decls.items() if n not in have]
        unexpected = [(n, self.source.shape(n)) for n in sorted(have - set(self.decls))]
        wrong = [(n, d.shapes, self.source.shape(n)) for n, d in self.decls.items()
                 if n in have and tuple(self.source.shape(n)) not in d.shapes]
        wrong += [(n, shapes, got) for n, shapes, got in self._conflicts]
        if missing or unexpected or wrong:
            raise WeightError(missing, unexpected, wrong)

    def fetch(self, name: str) -> torch.Tensor:
        if name in self._shared:
            return self._shared[name]
        decl = self.decls[name]
        t = self.source.tensor(name)
        target = memory_dtype(t.dtype, decl.role, self.rt.dtype)
        t = t.to(device=self.rt.device, dtype=target).reshape(decl.shapes[0]).contiguous()
        if self.uses[name] > 1:            # e.g. a table that is both embedding and head: one copy
            self._shared[name] = t
        return t

    def tensors_for(self, category: str, spec: PartSpec) -> dict[str, torch.Tensor]:
        decl = part_class(category, spec.kind).declare(spec.params)
        return {local: self.fetch(spec.tensors[local]) for local in decl}

    def release(self) -> None:
        self._shared.clear()


def expected_tensors(plan: ModelPlan) -> dict[str, TensorDecl]:
    """Checkpoint name -> declaration, for every tensor the plan reads."""
    from ..parts.model import plan_parts
    out = {}
    for category, spec in plan_parts(plan):
        for local, decl in part_class(category, spec.kind).declare(spec.params).items():
            out.setdefault(spec.tensors[local], decl)
    return out
