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
# Head size 64 (the tensor-core attention kernels and the tcgen05 prompt kernel), two layers of
# attention around a short convolution; used with sharpened attention (see ``sharpen_attention``).
TINY_C = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2",
    hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
    vocab_size=640, intermediate_size=256, block_auto_adjust_ff_dim=False, conv_L_cache=3, conv_bias=False,
    layer_types=["full_attention", "conv", "full_attention"], rope_theta=10000.0, norm_eps=1e-5,
    tie_embedding=True, max_position_embeddings=512,
)
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}


def make_folder(tmp, name: str, stored=torch.float32, gain_jitter=0.1, std=0.02):
    raw, seed = TINY[name]
    cfg = Lfm2Config.from_dict(raw)
    return write_random_model(Path(tmp) / f"tiny{name}_{str(stored).split('.')[-1]}", cfg, seed, dtype=stored,
                              gain_jitter=gain_jitter, std=std)


def sharpen_attention(folder, factor: float = 1.2):
    """Multiply the per-head q and k norm gains of a model folder by ``factor``: the scores'
    spread grows with its square (1.44 times at the default: scores of several units, a few keys
    carry most of the weight), so that a lost key, page or window edge changes the logits by
    far more than rounding.  The factor is kept moderate: rounding errors of the scores grow
    with the scores themselves, in 32-bit and above all in bfloat16."""
    from gibbs_b200.weights.safetensors_io import write_safetensors
    path = Path(folder) / "model.safetensors"
    raw = path.read_bytes()
    import struct
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    dtypes = {"F32": torch.float32, "BF16": torch.bfloat16}
    tensors = []
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + hlen + lo:8 + hlen + hi]), dtype=dtypes[info["dtype"]])
        t = t.reshape(info["shape"]).clone()
        if name.endswith(("q_layernorm.weight", "k_layernorm.weight")):
            t = (t.float() * factor).to(t.dtype)
        tensors.append((name, t))
    write_safetensors(path, iter(tensors), metadata=header.get("__metadata__", {}))
    return folder


def plain_logits(folder, ids) -> np.ndarray:
    cfg, w = plain.load_folder(folder)
    return plain.forward(cfg, w, ids).numpy()


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """Largest per-row relative L2 error."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    num = np.linalg.norm(got - want, axis=-1)
    den = np.linalg.norm(want, axis=-1) + 1e-30
    return float(np.max(num / den))


# Largest relative L2 error of a logits row against the float64 plain
# implementation.  float32: the engine measures 4e-7 to 5e-7 on both tiny models
# (2^-24 rounding accumulated over the products and layers); the bound leaves a
# factor of ten.  bfloat16: 2^-9 relative rounding of every activation, key and
# value that passes between kernels; the engine measures 4e-3 to 7e-3.
TOL = {"float32": 5e-6, "bfloat16": 2e-2}


def random_ids(seed: int, n: int, vocab: int) -> list[int]:
    g = np.random.default_rng(seed)
    return [int(v) for v in g.integers(0, vocab, n)]


# ---------------------------------------------------------------------------
# traces: lists of steps {"step", "entries": [{"id", "tokens", "want"}], "end"}
# ---------------------------------------------------------------------------

def trace_whole(requests: dict) -> list[dict]:
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(requests.items())]


def trace_tail_decoded(requests: dict, tail: int = 32) -> list[dict]:
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        head = max(len(ids) - tail, 1)
        steps.append({"entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        for t in range(head, len(ids)):
            steps.append({"entries": [{"id": rid, "tokens": [ids[t]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def trace_portions(requests: dict, sizes=(2, 3, 17, 2, 5, 16, 1, 31, 2, 64, 7)) -> list[dict]:
    """Each request alone, in portions of changing size, down to two tokens
    (and one, as a decoded token)."""
    steps = []
    for rid, ids in requests.items():
        pos, k = 0, 0
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            steps.append({"entries": [{"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))}], "end": []})
            pos, k = pos + n, k + 1
        steps[-1]["end"] = [rid]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def trace_mixed(requests: dict, capacity_tokens: int, max_live: int = 4, seed: int = 0, round_to: int = 64):
    """Up to ``max_live`` requests at a time; every step takes a random subset
    of them, portions of prompts for some beside single tokens for others;
    a request may sit a step out.  A request is admitted only while the live
    ones, each rounded up to ``round_to`` tokens, fit ``capacity_tokens`` —
    chosen small by the caller, so that pages and slots are used again."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: dict = {}
    steps = []

    def rounded(n):
        return -(-n // round_to) * round_to

    while waiting or live:
        while waiting and len(live) < max_live and \
                sum(rounded(len(v["ids"])) for v in live.values()) + rounded(len(waiting[0][1])) <= capacity_tokens:
            rid, ids = waiting.pop(0)
            live[rid] = {"ids": ids, "pos": 0}
        assert live, "capacity too small for the next request"
        chosen = [rid for rid in live if rng.random() < 0.75] or [next(iter(live))]
        entries, end = [], []
        for rid in chosen:
            st = live[rid]
            left = len(st["ids"]) - st["pos"]
            if left > 24 and rng.random() < 0.7:
                n = int(rng.integers(2, min(left - 8, 48) + 1))
            else:
                n = 1
            toks = st["ids"][st["pos"]:st["pos"] + n]
            entries.append({"id": rid, "tokens": toks, "want": list(range(n))})
            st["pos"] += n
            if st["pos"] == len(st["ids"]):
                end.append(rid)
        for rid in end:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def run_trace_on_engine(engine, steps) -> dict:
    """Drive Engine.step with a trace; returns {request id: [n_tokens, vocab] logits}."""
    from gibbs_b200 import StepEntry
    got: dict = {}
    for s in steps:
        entries = []
        for ent in s["entries"]:
            if not engine.is_live(ent["id"]):
                engine.open(ent["id"])
            entries.append(StepEntry(ent["id"], ent["tokens"], ent["want"]))
        logits = engine.step(entries)
        engine.check_status()
        if logits is not None:
            arr = logits.cpu().numpy()
            row = 0
            for ent in s["entries"]:
                base = engine.length(ent["id"]) - len(ent["tokens"])
                for w in ent["want"]:
                    got.setdefault(ent["id"], {})[base + w] = arr[row]
                    row += 1
        for rid in s["end"]:
            engine.close(rid)
        engine.cache.check()
    return {rid: np.stack([rows[p] for p in sorted(rows)]) for rid, rows in got.items()}


def first_wrong(got: np.ndarray, want: np.ndarray, tol: float):
    """Index of the first row whose relative error exceeds tol, or None."""
    num = np.linalg.norm(got.astype(np.float64) - want, axis=-1)
    den = np.linalg.norm(want, axis=-1) + 1e-30
    bad = np.nonzero(num / den > tol)[0]
    return None if bad.size == 0 else (int(bad[0]), float((num / den)[bad[0]]))
