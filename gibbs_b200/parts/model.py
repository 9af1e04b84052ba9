"""A causal language model assembled from a plan: embedding, blocks run in the
plan's order, final norm and head.  The same class serves every architecture;
what differs is the plan."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.plan import ModelPlan, PartSpec
from .base import Residual, Runtime, part_class, plan_ops_of


def plan_parts(plan: ModelPlan):
    """Every (category, spec) of a plan, in build order."""
    yield "embedding", plan.embedding
    for layer in plan.layers:
        yield "norm", layer.mixer_norm
        yield "mixer", layer.mixer
        yield "norm", layer.ffn_norm
        yield "feed_forward", layer.ffn
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
        return [(self.blocks[e.layer].mixer.cache_needs(), e.reads_cache_of) for e in self.plan.order]

    def kernel_libraries(self) -> set[str]:
        libs = {"core"}
        for part in [self.embedding, self.final_norm, self.head] + \
                [p for b in self.blocks for p in (b.mixer_norm, b.mixer, b.ffn_norm, b.ffn)]:
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
        z = self.final_norm.forward(x, rows=step.want_rows)
        return self.head.forward(z)

    def plan_ops(self, plan, caches) -> None:
        """Append everything ``forward`` does to a step plan; raises
        NotPlannable if a part cannot be written as operations."""
        plan_ops_of(self.embedding)(plan)
        for e, entry in enumerate(self.plan.order):
            plan_ops_of(self.blocks[entry.layer])(plan, caches[e])
        z = plan_ops_of(self.final_norm)(plan, wanted_rows=True)
        plan_ops_of(self.head)(plan, z, plan.LOGITS)

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads when each is read once: every
        projection matrix (a tied table once, as the head) and the small
        vectors; the embedding rows a step gathers are not counted."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor):
                    if v.data_ptr() not in seen and v.is_floating_point():
                        seen.add(v.data_ptr())
                        total += v.numel() * v.element_size()
                elif hasattr(v, "__dict__") and not isinstance(v, (Runtime, type)) and id(v) not in seen:
                    seen.add(id(v))
                    visit(v)

        for b in self.blocks:
            visit(b)
        visit(self.final_norm)
        visit(self.head)
        return total


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
    for layer in plan.layers:
        block_cls = part_class("block", layer.block)
        blocks.append(block_cls(make("norm", layer.mixer_norm), make("mixer", layer.mixer),
                                make("norm", layer.ffn_norm), make("feed_forward", layer.ffn), rt))
    final_norm = make("norm", plan.final_norm)
    head = make("head", plan.head)
    binder.release()
    return CausalLM(plan, rt, embedding, blocks, final_norm, head)
