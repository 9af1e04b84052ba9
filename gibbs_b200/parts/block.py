"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

from .base import Block, register_part


class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (MisterTK/gibbs arch/families/lfm2.json5:76-89)."""

    def forward(self, x, step, caches):
        h = self.mixer_norm.forward(x)
        self.mixer.forward(h, x, step, caches)
        h = self.ffn_norm.forward(x)
        self.ffn.forward(h, x, step)


register_part("block", "prenorm_residual", PreNormResidual)
