"""Token embedding and the output head."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorDecl, register_part
from .linear import Linear


class TokenEmbedding(Part):
    """x[t, :] = table[id_t, :], no scaling (MisterTK/gibbs arch/families/lfm2.json5:74)."""
    category = "embedding"

    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["vocab"], params["dim"])}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.vocab, self.dim = int(params["vocab"]), int(params["dim"])
        self.table = tensors["weight"].contiguous()

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(ids.numel(), self.dim, dtype=torch.float32)
        return ops.embed(self.table, ids, out)

    def plan_ops(self, plan):
        plan.embed(self.table)


class LMHead(Part):
    """logits = z W^T in 32-bit; with ``logit_scale`` they are divided by it, with
    ``softcap`` then passed through cap * tanh(x / cap)
    (MisterTK/gibbs arch/lib/transformer.json5:170-175; LFM2 has neither).  A
    tied head is given the embedding table's tensor and shares its memory."""
    category = "head"
    fuses_norm = True          # its input goes straight into a product (parts.linear.Linear)

    @classmethod
    def declare(cls, params):
        return {"weight": TensorDecl.of(params["vocab"], params["dim"])}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.vocab = int(params["vocab"])
        self.proj = Linear(tensors["weight"], None, rt)
        self.logit_scale = float(params.get("logit_scale", 1.0) or 1.0)
        self.softcap = float(params.get("softcap", 0.0) or 0.0)

    def kernel_libraries(self):
        return self.proj.kernel_libraries()

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        logits = self.proj(z, out_dtype=torch.float32)
        if self.logit_scale != 1.0 or self.softcap > 0.0:
            ops.scale_softcap(logits, 1.0 / self.logit_scale, self.softcap)
        return logits

    def plan_ops(self, plan, z, logits: int):
        """``logits``: the plan's symbol for where the step's float32 logits go."""
        plan.linear(z, self.proj.weight, self.proj.bias, logits, "plain", rows_symbol=plan.WANTED, role="lm_head")
        if self.logit_scale != 1.0 or self.softcap > 0.0:
            plan.scale_softcap(logits, self.vocab, plan.WANTED, 1.0 / self.logit_scale, self.softcap)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
