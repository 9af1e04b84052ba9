"""Random weights from a configuration and a seed: matrices, tables and biases
N(0, 0.02), norm gains 1.0 (optionally jittered, so that tests can tell a gain
from no gain).  Each tensor has its own generator seeded by (seed, name), so a
tensor's values do not depend on which other tensors exist.

MisterTK/gibbs has random weights only for synthetic llama ids
(``src/arch/load.rs:2355-2401``); the distribution here is the one this
project's benchmark configurations name.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Iterator

import torch

from ..config.plan import ModelPlan
from ..parts.base import VECTOR
from .loader import expected_tensors
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def _is_gain(name: str) -> bool:
    return name.endswith("norm.weight")


def random_tensors(plan: ModelPlan, seed: int, dtype: torch.dtype = torch.float32, std: float = 0.02,
                   gain_jitter: float = 0.0) -> Iterator[tuple[str, torch.Tensor]]:
    """(checkpoint name, tensor) for every tensor the plan reads, in the
    checkpoint's own shape, rounded to ``dtype``."""
    for name, decl in expected_tensors(plan).items():
        shape = decl.shapes[-1]            # the shape checkpoints of this architecture use
        g = torch.Generator().manual_seed(_seed_for(seed, name))
        if decl.role == VECTOR and _is_gain(name):
            t = torch.ones(shape)
            if gain_jitter:
                t = t + gain_jitter * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * std
        yield name, t.to(dtype)


def write_random_model(folder, config, seed: int, dtype: torch.dtype = torch.float32, std: float = 0.02,
                       gain_jitter: float = 0.0) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a typed configuration
    (anything with ``to_dict()`` and ``plan()``)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=1) + "\n")
    write_safetensors(folder / "model.safetensors",
                      random_tensors(config.plan(), seed, dtype, std, gain_jitter),
                      metadata={"format": "pt", "seed": seed})
    return folder
