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

    def lazy(self, x, rows=None):
        """Up to 16 rows of the stream in bfloat16: the product that reads them runs the
        norm itself (csrc/gemm_tc_decode.cu), with the sums of squares the product before
        left when there are some."""
        n = (x.shape[0] if rows is None else rows.numel())
        if (isinstance(x, Residual) and x.pending is None and ops.DECODE_PRODUCTS and ops.DECODE_NORM_INSIDE and self.rt.dtype == torch.bfloat16
                and n <= min(16, ops.DECODE_ROWS) and self.dim % 8 == 0 and x.x.stride(1) == 1 and x.x.stride(0) % 4 == 0
                and x.x.data_ptr() % 16 == 0):
            return ops.NormedRows(x.x, self.gain, self.eps, rows, x.ssq)
        return self.forward(x, rows=rows)

    def plan_ops(self, plan, wanted_rows: bool = False, lazy: bool = False):
        return plan.rmsnorm(self.gain, self.eps, wanted_rows, lazy=lazy)


register_part("norm", "rmsnorm", RMSNorm)
