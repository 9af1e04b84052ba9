"""Anchor of the plain implementation on the reference's own numbers.

MisterTK/gibbs is Rust; it cannot be compiled here (no cargo, no network), so
its model code is not run.  What it ships is a frozen LFM2 golden
(``tests/golden/lm_graphlm_lfm2.json`` there, copied verbatim beside this file
as ``ref_lfm2_golden.json``): five logit vectors and eight greedy ids of a
three-layer fixture whose weights come from a SplitMix64 stream
(``tests/golden/util.rs:19-85`` and ``tests/golden/lm.rs:262-309`` there).

This script regenerates that fixture as a model folder, runs
``tests/plain_lfm2.py`` on it and writes ``anchor_report.json`` (relative L2
error and cosine per golden vector, and the greedy ids).  Run it from the
repository root:  ``python tests/golden/make_anchor.py``.
"""
from __future__ import annotations

import json
import struct
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

MASK = (1 << 64) - 1

FIXTURE = dict(vocab=256, hidden=32, heads=4, kv=2, head_dim=8, inter=64, conv_k=3,
               layer_types=["conv", "full_attention", "conv"], seed=13)
PROMPT6 = [5, 17, 42, 99, 133, 200]
PROMPT20 = [(i * 37 + 11) % 252 + 4 for i in range(20)]
FORCED = [7, 64, 250]


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        return z ^ (z >> 31)

    def unit(self) -> np.float32:
        """Uniform in [-1, 1): top 24 bits / 2^24 * 2 - 1, in 32-bit arithmetic."""
        return np.float32(np.float32(self.next_u64() >> 40) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)


class FixtureWeights:
    def __init__(self, seed):
        self.rng = SplitMix64(seed)
        self.tensors: dict[str, np.ndarray] = {}

    def scaled(self, name, shape, scale):
        n = int(np.prod(shape))
        sc = np.float32(scale)
        self.tensors[name] = np.array([self.rng.unit() * sc for _ in range(n)], dtype=np.float32).reshape(shape)

    def matrix(self, name, shape):
        sc = np.float32(1.0) / np.sqrt(np.float32(shape[-1])) if len(shape) >= 2 else np.float32(0.5)
        self.scaled(name, shape, sc)

    def norm(self, name, n, center):
        self.tensors[name] = np.array(
            [np.float32(center) + self.rng.unit() * np.float32(0.1) for _ in range(n)], dtype=np.float32)


def fixture_config() -> dict:
    f = FIXTURE
    return {
        "model_type": "lfm2", "architectures": ["Lfm2ForCausalLM"], "vocab_size": f["vocab"],
        "hidden_size": f["hidden"], "num_hidden_layers": len(f["layer_types"]),
        "num_attention_heads": f["heads"], "num_key_value_heads": f["kv"], "head_dim": f["head_dim"],
        "intermediate_size": f["inter"], "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "hidden_act": "silu",
        "max_position_embeddings": 128, "bos_token_id": 1, "eos_token_id": 2, "tie_word_embeddings": True,
        "norm_eps": 1e-5, "conv_L_cache": f["conv_k"], "conv_bias": False,
        "block_auto_adjust_ff_dim": False, "layer_types": list(f["layer_types"]),
    }


def fixture_tensors() -> dict[str, np.ndarray]:
    f = FIXTURE
    h, hd = f["hidden"], f["head_dim"]
    a, kvd = f["heads"] * hd, f["kv"] * hd
    w = FixtureWeights(f["seed"])
    w.scaled("model.embed_tokens.weight", [f["vocab"], h], 0.05)
    w.norm("model.embedding_norm.weight", h, 1.0)
    for i, kind in enumerate(f["layer_types"]):
        p = f"model.layers.{i}"
        w.norm(p + ".operator_norm.weight", h, 1.0)
        w.norm(p + ".ffn_norm.weight", h, 1.0)
        if kind == "conv":
            w.matrix(p + ".conv.in_proj.weight", [3 * h, h])
            w.matrix(p + ".conv.conv.weight", [h, 1, f["conv_k"]])
            w.matrix(p + ".conv.out_proj.weight", [h, h])
        else:
            w.matrix(p + ".self_attn.q_proj.weight", [a, h])
            w.matrix(p + ".self_attn.k_proj.weight", [kvd, h])
            w.matrix(p + ".self_attn.v_proj.weight", [kvd, h])
            w.matrix(p + ".self_attn.out_proj.weight", [h, a])
            w.norm(p + ".self_attn.q_layernorm.weight", hd, 1.0)
            w.norm(p + ".self_attn.k_layernorm.weight", hd, 1.0)
        w.matrix(p + ".feed_forward.w1.weight", [f["inter"], h])
        w.matrix(p + ".feed_forward.w3.weight", [f["inter"], h])
        w.matrix(p + ".feed_forward.w2.weight", [h, f["inter"]])
    return w.tensors


def write_safetensors_f32(path, tensors: dict[str, np.ndarray]):
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        b = np.ascontiguousarray(arr, dtype="<f4").tobytes()
        header[name] = {"dtype": "F32", "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(hj)))
        fh.write(hj)
        for b in blobs:
            fh.write(b)


def write_fixture(folder):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(fixture_config(), indent=1))
    write_safetensors_f32(folder / "model.safetensors", fixture_tensors())
    return folder


def golden() -> dict:
    return json.loads((HERE / "ref_lfm2_golden.json").read_text())


def golden_cases():
    """(name, token ids whose last-row logits the golden vector holds)."""
    cases = [("prefill6", PROMPT6), ("prefill20", PROMPT20)]
    for i in range(3):
        cases.append((f"decode{i}", PROMPT6 + FORCED[: i + 1]))
    return cases


def main():
    import plain_lfm2 as plain

    ref = golden()
    with tempfile.TemporaryDirectory() as tmp:
        cfg, weights = plain.load_folder(write_fixture(tmp))
    report = {"source": "tests/golden/lm_graphlm_lfm2.json of MisterTK/gibbs", "cases": {}}
    for name, ids in golden_cases():
        got = plain.forward(cfg, weights, ids)[-1].numpy()
        want = np.array(ref["f32"][name], dtype=np.float64)
        rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        cos = float(got @ want / (np.linalg.norm(got) * np.linalg.norm(want)))
        report["cases"][name] = {"rel_l2": rel, "cosine": cos, "max_abs": float(np.abs(got - want).max())}
    ids = plain.greedy(cfg, weights, PROMPT6, 8)
    report["greedy8"] = {"plain": ids, "reference": ref["ids"]["greedy8"]}
    (HERE / "anchor_report.json").write_text(json.dumps(report, indent=1) + "\n")
    print(json.dumps(report, indent=1))


if __name__ == "__main__":
    main()
