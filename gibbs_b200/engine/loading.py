"""From a model folder (config.json + safetensors) to a model on the GPU."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from ..config import parse_config
from ..parts.model import CausalLM, build_model
from ..weights import Checkpoint, TensorDict, random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype {name}: the engine computes in bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype '{name}'; use bfloat16 or float32") from None


def load_model(folder, dtype="bfloat16", device="cuda:0", arch: Optional[str] = None) -> CausalLM:
    """Read config.json, pick the architecture it names, check the checkpoint
    against the resulting plan and build the model on ``device``."""
    folder = Path(folder)
    cfg_path = folder / "config.json"
    if not cfg_path.exists():
        raise FileNotFoundError(f"{folder} has no config.json")
    cfg = json.loads(cfg_path.read_text())
    ckpt = Checkpoint(folder)
    conf = parse_config(cfg, ckpt.names(), forced=arch)
    model = build_model(conf.plan(), ckpt, parse_dtype(dtype), device)
    model.config = conf
    return model


def random_model(config, seed: int, dtype="bfloat16", device="cuda:0", stored_dtype=None,
                 gain_jitter: float = 0.0) -> CausalLM:
    """A model with the random weights ``write_random_model`` would write for
    (config, seed), built without going through a file."""
    dt = parse_dtype(dtype)
    tensors = dict(random_tensors(config.plan(), seed, stored_dtype or dt, gain_jitter=gain_jitter))
    model = build_model(config.plan(), TensorDict(tensors), dt, device)
    model.config = config
    return model
