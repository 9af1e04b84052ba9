"""A causal language model assembled from a plan: embedding, blocks run in the
plan's order, final norm and head.  The same class serves every architecture;
what differs is the plan."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.plan import ModelPlan, PartSpec
from .base import Residual, Runtime, part_class, plan_ops_of, step_weight_bytes


def plan_parts(plan: ModelPlan):
    """Every (category, spec) of a plan, in build order."""
    yield "embedding", plan.embedding
    for layer in plan.layers:
        for _, category, spec in layer.parts:
            yield category, spec
    yield "norm", plan.final_norm
    yield "head", plan.head


class CausalLM:
    def __init__(self, plan: ModelPlan, rt: Runtime, embedding, blocks, final_norm, head):
        self.plan, self.rt = plan, rt
        self.embedding, self.blocks, self.final_norm, self.head = embedding, blocks, final_norm, head
        self.vocab_size, self.hidden_size = plan.vocab_size, plan.hidden_size

    def entry_needs(self):
        """For each entry of the plan's order: (cache needs of its mixer, the
        entry whose cache it reads instead, or None)."""
        return [(self.blocks[e.layer].cache_needs(), e.reads_cache_of) for e in self.plan.order]

    def kernel_libraries(self) -> set[str]:
        libs = {"core"}
        for part in [self.embedding, self.final_norm, self.head] + \
                [p for b in self.blocks for p in b.parts.values()]:
            libs |= set(part.kernel_libraries())
        return libs

    def forward(self, step, caches) -> Optional[torch.Tensor]:
        """Run the step's tokens through every entry of the order; return the
        32-bit logits of the wanted rows, [n_want, vocab], or None."""
        x = Residual(self.embedding.forward(step.token_ids))
        for e, entry in enumerate(self.plan.order):
            self.blocks[entry.layer].forward(x, step, caches[e])
        if step.n_want == 0:
            return None
        if getattr(self.head, "fuses_norm", False):
            z = self.final_norm.lazy(x, rows=step.want_rows)
        else:
            z = self.final_norm.forward(x, rows=step.want_rows)
        return self.head.forward(z)

    def plan_ops(self, plan, caches) -> None:
        """Append everything ``forward`` does to a step plan; raises
        NotPlannable if a part cannot be written as operations."""
        plan_ops_of(self.embedding)(plan)
        for e, entry in enumerate(self.plan.order):
            plan_ops_of(self.blocks[entry.layer])(plan, caches[e])
        if getattr(self.head, "fuses_norm", False) and getattr(self.final_norm, "lazy", None) is not None:
            try:
                z = plan_ops_of(self.final_norm)(plan, wanted_rows=True, lazy=True)
            except TypeError:            # a norm from outside whose plan_ops knows no such option
                z = plan_ops_of(self.final_norm)(plan, wanted_rows=True)
        else:
            z = plan_ops_of(self.final_norm)(plan, wanted_rows=True)
        plan_ops_of(self.head)(plan, z, plan.LOGITS)

    def weight_bytes_per_step(self, n_tokens: int = 1) -> int:
        """Bytes of weights a step of ``n_tokens`` tokens reads when each is
        read once: every projection matrix (a tied table once, as the head)
        and the small vectors; the embedding rows a step gathers are not
        counted.  Each part answers for itself (``parts.base.step_weight_bytes``)."""
        seen: set = set()
        total = 0
        for b in self.blocks:
            for part in b.parts.values():
                total += step_weight_bytes(part, n_tokens, seen)
        return total + step_weight_bytes(self.final_norm, n_tokens, seen) + step_weight_bytes(self.head, n_tokens, seen)


def build_model(plan: ModelPlan, source, dtype: torch.dtype, device) -> CausalLM:
    """Check ``source`` (a Checkpoint or TensorDict) against the plan, then
    build every part with its tensors on ``device``."""
    from ..weights.loader import WeightBinder

    plan.validate()
    rt = Runtime(dtype=dtype, device=torch.device(device))
    binder = WeightBinder(plan, source, rt)
    binder.verify()

    def make(category: str, spec: PartSpec):
        cls = part_class(category, spec.kind)
        return cls(spec.params, binder.tensors_for(category, spec), rt)

    embedding = make("embedding", plan.embedding)
    blocks = []
    for i, layer in enumerate(plan.layers):
        block_cls = part_class("block", layer.block)
        given = tuple((role, category) for role, category, _ in layer.parts)
        wanted = tuple(getattr(block_cls, "ROLES", ()))
        if wanted and given != wanted:
            raise ValueError(f"layer {i}: the '{layer.block}' arrangement is made of {list(wanted)}; "
                             f"the plan gives {list(given)}")
        blocks.append(block_cls({role: make(category, spec) for role, category, spec in layer.parts}, rt,
                                layer.params))
    final_norm = make("norm", plan.final_norm)
    head = make("head", plan.head)
    binder.release()
    return CausalLM(plan, rt, embedding, blocks, final_norm, head)
