"""Shared by the tests: the two tiny configurations, model folders made in a
temporary place, and the comparison of engine logits with the plain
implementation."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_lfm2 as plain
from gibbs_b200 import Lfm2Config
from gibbs_b200.weights import write_random_model

# Two tiny configurations that differ in every size and option.
TINY_A = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2",
    hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    vocab_size=512, intermediate_size=192, block_auto_adjust_ff_dim=False, conv_L_cache=3, conv_bias=False,
    layer_types=["conv", "full_attention", "conv", "full_attention"], rope_theta=10000.0, norm_eps=1e-5,
    tie_embedding=True, max_position_embeddings=512,
)
TINY_B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2",
    hidden_size=96, num_hidden_layers=6, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
    vocab_size=1000, intermediate_size=384, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
    block_multiple_of=64, conv_L_cache=4, conv_bias=True, attention_bias=True,
    full_attn_idxs=[0, 2, 5], rope_theta=1000000.0, norm_eps=1e-6,
    tie_embedding=False, max_position_embeddings=512,
)
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1)}


def make_folder(tmp, name: str, stored=torch.float32, gain_jitter=0.1, std=0.02):
    raw, seed = TINY[name]
    cfg = Lfm2Config.from_dict(raw)
    return write_random_model(Path(tmp) / f"tiny{name}_{str(stored).split('.')[-1]}", cfg, seed, dtype=stored,
                              gain_jitter=gain_jitter, std=std)


def plain_logits(folder, ids) -> np.ndarray:
    cfg, w = plain.load_folder(folder)
    return plain.forward(cfg, w, ids).numpy()


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """Largest per-row relative L2 error."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    num = np.linalg.norm(got - want, axis=-1)
    den = np.linalg.norm(want, axis=-1) + 1e-30
    return float(np.max(num / den))


# Relative L2 error per logits row against the float64 plain implementation.
# float32: accumulated rounding of 2^-24 over a few thousand fused multiply-adds
# per element and a few layers.  bfloat16: 2^-8 per rounding of activations, keys
# and values between kernels, over the layers of the tiny models.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def random_ids(seed: int, n: int, vocab: int) -> list[int]:
    g = np.random.default_rng(seed)
    return [int(v) for v in g.integers(0, vocab, n)]
