"""Position encodings.  Rotary encodings hand their table to the mixer, whose
kernel applies it to q and k together with the per-head norm."""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, Rotary, register_part


def _inv_freq_f32(rotary_dim: int, theta: float) -> np.ndarray:
    """inv_freq[j] = 1 / theta^(2j / rotary_dim), every step in 32-bit
    (MisterTK/gibbs src/arch/gen.rs:137-164, precision 'f32';
    arch/families/lfm2.json5:63-65)."""
    j = np.arange(rotary_dim // 2, dtype=np.float32)
    expo = (np.float32(2.0) * j) / np.float32(rotary_dim)
    return (np.float32(1.0) / np.power(np.float32(theta), expo, dtype=np.float32)).astype(np.float32)


class RotaryHalfSplit(PositionEncoding):
    """Rotates the pairs (j, j + rotary_dim/2) by pos * inv_freq[j]
    (MisterTK/gibbs src/graph/cpu.rs:688-697)."""
    adjacent = False

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.inv_freq = torch.from_numpy(_inv_freq_f32(self.rotary_dim, float(params["theta"]))).to(rt.device)
        # the factor on cosines and sines (MisterTK/gibbs src/graph/cpu.rs:674-675); 1 unless given
        self._rotary = Rotary(self.inv_freq, self.rotary_dim, self.adjacent, float(params.get("mscale", 1.0)))

    def rotary(self):
        return self._rotary


class RotaryAdjacent(RotaryHalfSplit):
    """Rotates the pairs (2j, 2j + 1) (MisterTK/gibbs src/graph/cpu.rs:678-687)."""
    adjacent = True


class NoPosition(PositionEncoding):
    pass


register_part("position", "rope_half_split", RotaryHalfSplit)
register_part("position", "rope_adjacent", RotaryAdjacent)
register_part("position", "none", NoPosition)
