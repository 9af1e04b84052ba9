"""Gated short convolution: [B; C; x] = in_proj(h); out_proj(C * conv(B * x))
with a depthwise causal convolution of width ``kernel`` whose last
``kernel - 1`` inputs are the request's fixed-size state
(MisterTK/gibbs arch/lib/transformer.json5:140-151; src/graph/cpu.rs:952-994).
A depthwise bias (refused by the reference, arch/families/lfm2.json5:53) adds
to the convolution before the C gate."""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, SlotState, TensorDecl, VECTOR, register_part
from .linear import Linear


class GatedShortConv(Mixer):
    fuses_norm = True          # its input goes straight into a product (parts.linear.Linear)

    @classmethod
    def declare(cls, params):
        h, k = params["hidden"], params["kernel"]
        d = {
            "in_proj.weight": TensorDecl.of(3 * h, h),
            "conv.weight": TensorDecl(((h, k), (h, 1, k)), VECTOR),
            "out_proj.weight": TensorDecl.of(h, h),
        }
        if params.get("bias"):
            d["in_proj.bias"] = TensorDecl.of(3 * h, role=VECTOR)
            d["conv.bias"] = TensorDecl.of(h, role=VECTOR)
            d["out_proj.bias"] = TensorDecl.of(h, role=VECTOR)
        return d

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hidden, self.kernel = int(params["hidden"]), int(params["kernel"])
        if self.kernel < 2:
            raise ValueError(f"short-conv kernel width {self.kernel} must be >= 2")
        self.in_proj = Linear(tensors["in_proj.weight"], tensors.get("in_proj.bias"), rt)
        self.out_proj = Linear(tensors["out_proj.weight"], tensors.get("out_proj.bias"), rt)
        self.taps = tensors["conv.weight"].to(torch.float32).reshape(self.hidden, self.kernel).contiguous()
        cb = tensors.get("conv.bias")
        self.conv_bias = None if cb is None else cb.to(torch.float32).contiguous()

    def kernel_libraries(self):
        return tuple(set(self.in_proj.kernel_libraries()) | set(self.out_proj.kernel_libraries()) | {"core"})

    def cache_needs(self):
        return [SlotState((self.kernel - 1, self.hidden), torch.float32)]

    def forward(self, h, residual, step, caches):
        slot = caches[0]
        y = self.rt.empty(h.shape[0], self.hidden)
        one_each = step.max_q_len == 1 and step.n_tokens == step.n_requests
        bcx = self.in_proj.partials(h) if one_each else self.in_proj(h)
        if isinstance(bcx, ops.Partials):
            ops.short_conv_partials(bcx, self.taps, self.conv_bias, slot.state, slot.slot_ids, step.q_start, y)
        else:
            ops.short_conv(bcx, self.taps, self.conv_bias, slot.state, slot.slot_ids, step.tok_req, step.q_start,
                           step.q_len, y, max_q_len=step.max_q_len)
        self.out_proj(y, out=residual, accumulate=True)

    def plan_ops(self, plan, h, caches):
        bcx = plan.linear(h, self.in_proj.weight, self.in_proj.bias, plan.buffer("bcx", 3 * self.hidden), "plain",
                          partials="one_each", role="in_proj")
        y = plan.short_conv(bcx, self.taps, self.conv_bias, caches[0], self.hidden, self.kernel)
        plan.linear(y, self.out_proj.weight, self.out_proj.bias, None, "residual", role="out_proj")


register_part("mixer", "gated_short_conv", GatedShortConv)
