"""RMSNorm: x * (1/sqrt(mean(x^2) + eps)) * gain, statistics in 32-bit
(MisterTK/gibbs arch/lib/transformer.json5:9-11; src/model/simd.rs:73-111)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, Residual, TensorDecl, VECTOR, register_part


class RMSNorm(Norm):
    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["dim"], role=VECTOR)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.dim, self.eps = int(params["dim"]), float(params["eps"])
        self.gain = tensors["weight"].to(torch.float32).contiguous()

    def forward(self, x, out=None, rows=None):
        pending = None
        if isinstance(x, Residual):
            pending, x = x.take_pending(), x.x
        n = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = self.rt.empty(n, self.dim)
        return ops.rmsnorm(x, self.gain, self.eps, out, rows, pending)


    def plan_ops(self, plan, wanted_rows: bool = False):
        return plan.rmsnorm(self.gain, self.eps, wanted_rows)


register_part("norm", "rmsnorm", RMSNorm)
