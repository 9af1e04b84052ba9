"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

from .base import Block, plan_ops_of, register_part


class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (MisterTK/gibbs arch/families/lfm2.json5:76-89)."""
    ROLES = (("mixer_norm", "norm"), ("mixer", "mixer"), ("ffn_norm", "norm"), ("ffn", "feed_forward"))

    # A mixer or feed-forward that says ``fuses_norm`` hands its input straight to a product
    # (``parts.linear.Linear``), which may then run the norm itself.

    def forward(self, x, step, caches):
        h = self.mixer_norm.lazy(x) if getattr(self.mixer, "fuses_norm", False) else self.mixer_norm.forward(x)
        self.mixer.forward(h, x, step, self.caches_of("mixer", caches))
        h = self.ffn_norm.lazy(x) if getattr(self.ffn, "fuses_norm", False) else self.ffn_norm.forward(x)
        self.ffn.forward(h, x, step)

    def plan_ops(self, plan, caches):
        h = self._norm_ops(plan, self.mixer_norm, self.mixer)
        plan_ops_of(self.mixer)(plan, h, self.caches_of("mixer", caches))
        h = self._norm_ops(plan, self.ffn_norm, self.ffn)
        plan_ops_of(self.ffn)(plan, h)

    @staticmethod
    def _norm_ops(plan, norm, consumer):
        if getattr(consumer, "fuses_norm", False) and getattr(norm, "lazy", None) is not None:
            try:
                return plan_ops_of(norm)(plan, lazy=True)
            except TypeError:            # a norm from outside whose plan_ops knows no such option
                pass
        return plan_ops_of(norm)(plan)


register_part("block", "prenorm_residual", PreNormResidual)
