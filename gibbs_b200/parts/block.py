"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

from .base import Block, plan_ops_of, register_part


class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (MisterTK/gibbs arch/families/lfm2.json5:76-89)."""
    ROLES = (("mixer_norm", "norm"), ("mixer", "mixer"), ("ffn_norm", "norm"), ("ffn", "feed_forward"))

    def forward(self, x, step, caches):
        h = self.mixer_norm.forward(x)
        self.mixer.forward(h, x, step, self.caches_of("mixer", caches))
        h = self.ffn_norm.forward(x)
        self.ffn.forward(h, x, step)

    def plan_ops(self, plan, caches):
        h = plan_ops_of(self.mixer_norm)(plan)
        plan_ops_of(self.mixer)(plan, h, self.caches_of("mixer", caches))
        h = plan_ops_of(self.ffn_norm)(plan)
        plan_ops_of(self.ffn)(plan, h)


register_part("block", "prenorm_residual", PreNormResidual)
