"""SwiGLU feed-forward: down((g * sigmoid(g)) * u), g = gate(h), u = up(h)
(MisterTK/gibbs arch/lib/transformer.json5:117-130; src/graph/cpu.rs:378-390).
Gate and up are one fused product."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorDecl, VECTOR, register_part
from .linear import Linear, can_fuse_swiglu, interleave_gate_up


class SwiGLU(FeedForward):
    fuses_norm = True          # its input goes straight into a product (parts.linear.Linear)

    @classmethod
    def declare(cls, params):
        h, f = params["hidden"], params["inner"]
        d = {"gate.weight": TensorDecl.of(f, h), "up.weight": TensorDecl.of(f, h), "down.weight": TensorDecl.of(h, f)}
        if params.get("bias"):
            d.update({"gate.bias": TensorDecl.of(f, role=VECTOR), "up.bias": TensorDecl.of(f, role=VECTOR),
                      "down.bias": TensorDecl.of(h, role=VECTOR)})
        return d

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hidden, self.inner = int(params["hidden"]), int(params["inner"])
        if tensors["gate.weight"].dtype != tensors["up.weight"].dtype:
            raise ValueError("gate and up projections are stored in different dtypes")
        self.fused = can_fuse_swiglu(tensors["gate.weight"], rt)
        join = interleave_gate_up if self.fused else (lambda g, u: torch.cat([g, u], 0))
        w = join(tensors["gate.weight"], tensors["up.weight"])
        b = None
        if params.get("bias"):
            b = join(tensors["gate.bias"].to(torch.float32), tensors["up.bias"].to(torch.float32))
        self.gate_up = Linear(w, b, rt, swiglu=self.fused)
        self.down = Linear(tensors["down.weight"], tensors.get("down.bias"), rt)

    def kernel_libraries(self):
        return tuple(set(self.gate_up.kernel_libraries()) | set(self.down.kernel_libraries()) | {"core"})

    def forward(self, h, residual, step):
        if self.fused:
            act = self.gate_up(h)
        else:
            gu = self.gate_up(h)
            act = self.rt.empty(h.shape[0], self.inner)
            ops.swiglu(gu, act)
        self.down(act, out=residual, accumulate=True)

    def plan_ops(self, plan, h):
        gu = self.gate_up
        if self.fused:
            act = plan.linear(h, gu.weight, gu.bias, plan.buffer("act", self.inner), "swiglu", role="gate_up")
        else:
            both = plan.linear(h, gu.weight, gu.bias, plan.buffer("gate_up", 2 * self.inner), "plain", role="gate_up")
            act = plan.swiglu(both, self.inner)
        plan.linear(act, self.down.weight, self.down.bias, None, "residual", role="down")


register_part("feed_forward", "swiglu", SwiGLU)
