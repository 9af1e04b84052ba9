"""A dense projection y = x W^T (+ b): a helper the parts share, not a part of
its own.  It owns the choice of matrix-product kernel for its operand types."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Residual, Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], rt: Runtime, swiglu: bool = False):
        """``swiglu``: the weight holds gate and up rows alternating in blocks
        of 64 and calls return (g * sigmoid(g)) * u (see ``interleave_gate_up``)."""
        self.weight = weight.contiguous()          # [out, in], as stored (bfloat16 or float32)
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.out_features, self.in_features = self.weight.shape
        if swiglu:
            self.out_features //= 2
        self.swiglu = swiglu
        self.rt = rt

    def kernel_libraries(self):
        return ops.linear_libraries(self.weight.dtype, self.rt.dtype)

    def _decode(self, x) -> bool:
        """Whether this call runs on the decode kernel (up to 64 rows, cluster split-K)."""
        if self.rt.dtype != torch.bfloat16 or x.shape[0] > ops.DECODE_ROWS \
                or not ops.linear_decode_supported(x.shape[0], self.weight):
            return False
        if isinstance(x, ops.NormedRows):
            return True                 # (whether the norm runs inside is asked in __call__)
        return (x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)

    def partials(self, x):
        """x W^T + b for a consumer that can add split-K partial tiles itself:
        ``ops.Partials`` when the product runs on the tensor cores with K split
        (then no reduction kernel runs), else the finished product."""
        if self._decode(x):
            return self(x)
        if isinstance(x, ops.NormedRows):
            x = x.tensor()
        if not self.swiglu and self.rt.dtype == torch.bfloat16 and ops.linear_tc_supported(x, self.weight):
            return ops.linear_tc_partials(x, self.weight, self.bias)
        return self(x)

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """out (+)= x W^T + b.  ``accumulate`` adds into a float32 ``out``
        (the residual stream)."""
        decode = self._decode(x)
        if isinstance(x, ops.NormedRows) and not (decode and ops.linear_decode_normed_ok(x.shape[0], *self.weight.shape)):
            x = x.tensor()                      # this product cannot take the norm in: the norm runs by itself
            decode = self._decode(x)
        if isinstance(out, Residual):
            if not accumulate:
                raise ValueError("a projection can only add into the residual stream")
            if decode:
                out.ssq = ops.linear_decode(x, self.weight, self.bias, out.tensor(), accumulate=True, want_ssq=True)
                return out
            if ops.linear_tc_supported(x, self.weight):
                res = ops.linear_tc(x, self.weight, self.bias, out.tensor(), accumulate=True,
                                    defer=True)
                if res is not out.x:              # K was split: the next norm adds the partial sums
                    out.defer(res, self.bias)
                return out
            ops.linear(x, self.weight, self.bias, out.tensor(), True)
            return out
        if out is None:
            out = torch.empty(x.shape[0], self.out_features, dtype=out_dtype or self.rt.dtype, device=x.device)
        if decode:
            ops.linear_decode(x, self.weight, self.bias, out, accumulate=accumulate, swiglu=self.swiglu)
            return out
        if self.swiglu:
            return ops.linear_tc(x, self.weight, self.bias, out, swiglu=True)
        return ops.linear(x, self.weight, self.bias, out, accumulate)


def can_fuse_swiglu(gate: torch.Tensor, rt: Runtime) -> bool:
    """Whether gate/up of this shape run as one product with the SwiGLU epilogue."""
    inner, hidden = gate.shape
    return gate.dtype == torch.bfloat16 and rt.dtype == torch.bfloat16 and inner % 64 == 0 and hidden % 8 == 0


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate rows 0..63; up rows 0..63; gate rows 64..127; up rows 64..127; ...]:
    each 128-row tile of the product then holds g and u of the same 64 features."""
    inner = gate.shape[0]
    g = gate.reshape(inner // 64, 64, *gate.shape[1:])
    u = up.reshape(inner // 64, 64, *up.shape[1:])
    return torch.stack([g, u], 1).reshape(2 * inner, *gate.shape[1:]).contiguous()
