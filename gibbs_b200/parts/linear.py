"""A dense projection y = x W^T (+ b): a helper the parts share, not a part of
its own.  It owns the choice of matrix-product kernel for its operand types."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], rt: Runtime):
        self.weight = weight.contiguous()          # [out, in], as stored (bfloat16 or float32)
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.rt = rt

    def kernel_libraries(self):
        return ops.linear_libraries(self.weight.dtype, self.rt.dtype)

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """out (+)= x W^T + b.  ``accumulate`` adds into a float32 ``out``
        (the residual stream)."""
        if out is None:
            out = torch.empty(x.shape[0], self.out_features, dtype=out_dtype or self.rt.dtype, device=x.device)
        return ops.linear(x, self.weight, self.bias, out, accumulate)
