"""Plain, slow LFM2 forward pass: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the product
path (``gibbs_b200``): it reads ``config.json`` and the safetensors file itself
and computes every formula in the precision it is given (float64 by default).
Every function cites the place in MisterTK/gibbs where the formula was read
(paths are relative to that project's root).

The reference's own model code is Rust and cannot be compiled in this
environment, so the functions below rest on its formulas; they are anchored
once against the reference's frozen LFM2 golden logits
(``tests/golden/lm_graphlm_lfm2.json`` of the reference, copied to
``tests/golden/ref_lfm2_golden.json`` here) by ``tests/golden/make_anchor.py``.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ----------------------------------------------------------------------------
# checkpoint reading (independent of gibbs_b200.weights)
# ----------------------------------------------------------------------------

_NP_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, payload
    (src/model/mod.rs:398-410)."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[base + lo : base + hi]
        shape = info["shape"]
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32)
        else:
            arr = np.frombuffer(buf, dtype=_NP_DTYPES[info["dtype"]])
        out[name] = torch.from_numpy(arr.astype(np.float64).reshape(shape))
    return out


def load_folder(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = read_safetensors(folder / "model.safetensors")
    return cfg, weights


# ----------------------------------------------------------------------------
# configuration (arch/families/lfm2.json5:27-51)
# ----------------------------------------------------------------------------

def first(*vals):
    for v in vals:
        if v is not None:
            return v
    return None


def resolve_sizes(cfg: dict) -> dict:
    """The numbers the LFM2 family spec derives from config.json
    (arch/families/lfm2.json5:27-51)."""
    hidden = cfg["hidden_size"]
    heads = first(cfg.get("num_attention_heads"), cfg.get("num_heads"))
    kv_heads = first(cfg.get("num_key_value_heads"), heads)
    head_dim = first(cfg.get("head_dim"), hidden // heads)
    ff_raw = first(cfg.get("intermediate_size"), cfg.get("block_ff_dim"), 4 * hidden)
    ff_23 = ff_raw * 2 // 3
    mult_of = first(cfg.get("block_multiple_of"), 256)
    if cfg.get("block_auto_adjust_ff_dim") is True:
        m = first(cfg.get("block_ffn_dim_multiplier"), 0)
        inter = mult_of * math.ceil(int(m * ff_23) / mult_of) if m > 0 else ff_23
    else:
        inter = ff_raw
    rope = cfg.get("rope_parameters") or {}
    return dict(
        hidden=hidden,
        layers=cfg["num_hidden_layers"],
        heads=heads,
        kv_heads=kv_heads,
        head_dim=head_dim,
        inter=inter,
        eps=first(cfg.get("norm_eps"), cfg.get("rms_norm_eps"), 1e-5),
        theta=first(cfg.get("rope_theta"), rope.get("rope_theta"), 10000),
        conv_k=cfg["conv_L_cache"],
    )


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def rms_norm(x, gain, eps):
    """out = x * (1/sqrt(mean(x^2) + eps)) * gain over the last axis, which has
    the gain's length (src/model/simd.rs:73-111, src/graph/cpu.rs:358-377)."""
    scale = 1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return x * scale * gain


def linear(x, weight, bias=None):
    """y = x W^T (+ b) (arch/lib/transformer.json5:50-54; src/graph/cpu.rs:249-274)."""
    y = x @ weight.T
    return y if bias is None else y + bias


def rope_inv_freq(head_dim, theta, dtype):
    """inv_freq[j] = 1 / theta^(2j/head_dim), generated in 32-bit
    (arch/families/lfm2.json5:63-65; src/arch/gen.rs:137-164)."""
    j = np.arange(head_dim // 2, dtype=np.float32)
    inv = np.float32(1.0) / np.power(np.float32(theta), (np.float32(2.0) * j) / np.float32(head_dim), dtype=np.float32)
    return torch.from_numpy(inv.astype(np.float32)).to(dtype)


def rope_half_split(x, positions, inv_freq):
    """Pairs (j, j + hd/2): out[j] = x[j] cos - x[j+hd/2] sin,
    out[j+hd/2] = x[j] sin + x[j+hd/2] cos with angle = pos * inv_freq[j]
    (src/graph/cpu.rs:632-697, HalfSplit).  x: [n, heads, hd]."""
    half = x.shape[-1] // 2
    # the reference forms the angle in 32-bit: (p as f32) * freq (src/graph/cpu.rs:673)
    ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(x.dtype)
    c = torch.cos(ang)[:, None, :]
    s = torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def causal_attention(q, k, v, scale, window=None):
    """Softmax((q.k) * scale) over keys j <= p (and j + window > p when a
    window is set), max subtracted, masked keys weigh 0; query head h reads
    kv head h // (heads/kv_heads) (src/graph/cpu.rs:826-951).
    q: [n, heads, hd]; k, v: [n, kv_heads, hd]."""
    n, heads, hd = q.shape
    rep = heads // k.shape[1]
    out = torch.zeros_like(q)
    idx = torch.arange(n, device=q.device)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask &= idx[None, :] + window > idx[:, None]
    for h in range(heads):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        s = torch.where(mask, s, torch.full_like(s, float("-inf")))
        w = torch.exp(s - s.max(-1, keepdim=True).values)
        w = w / w.sum(-1, keepdim=True)
        out[:, h] = w @ v[:, h // rep]
    return out


def attention_mixer(h, w, prefix, sizes, positions):
    """q/k/v projections (bias by presence), per-head RMSNorm of q and k
    before RoPE with the layer eps, half-split RoPE, causal GQA attention with
    scale 1/sqrt(head_dim), output projection
    (arch/lib/transformer.json5:46-87; arch/families/lfm2.json5:45-48, 80-83)."""
    n = h.shape[0]
    heads, kvh, hd = sizes["heads"], sizes["kv_heads"], sizes["head_dim"]
    q = linear(h, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).reshape(n, heads, hd)
    k = linear(h, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).reshape(n, kvh, hd)
    v = linear(h, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).reshape(n, kvh, hd)
    q = rms_norm(q, w[prefix + "q_layernorm.weight"], sizes["eps"])
    k = rms_norm(k, w[prefix + "k_layernorm.weight"], sizes["eps"])
    inv = rope_inv_freq(hd, sizes["theta"], h.dtype).to(h.device)
    q = rope_half_split(q, positions, inv)
    k = rope_half_split(k, positions, inv)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(hd))
    return linear(o.reshape(n, heads * hd), w[prefix + "out_proj.weight"], w.get(prefix + "out_proj.bias"))


def causal_conv1d(bx, taps, bias=None):
    """Depthwise causal conv over [zeros(K-1); bx]: tap K-1 multiplies the
    current row, tap 0 the oldest (src/graph/cpu.rs:952-994).
    bx: [n, C]; taps: [C, K].  A depthwise bias, which the reference refuses
    (arch/families/lfm2.json5:53), adds to the conv output."""
    n, _ = bx.shape
    kk = taps.shape[1]
    pad = torch.cat([torch.zeros(kk - 1, bx.shape[1], dtype=bx.dtype, device=bx.device), bx], 0)
    out = torch.zeros_like(bx)
    for j in range(kk):
        out = out + pad[j : j + n] * taps[:, j][None, :]
    return out if bias is None else out + bias[None, :]


def short_conv_mixer(h, w, prefix, sizes):
    """[B; C; x] = in_proj(h); out_proj(C * conv(B * x))
    (arch/lib/transformer.json5:140-151)."""
    hid = sizes["hidden"]
    bcx = linear(h, w[prefix + "in_proj.weight"], w.get(prefix + "in_proj.bias"))
    b, c, xs = bcx[:, :hid], bcx[:, hid : 2 * hid], bcx[:, 2 * hid :]
    taps = w[prefix + "conv.weight"].reshape(hid, sizes["conv_k"])
    cv = causal_conv1d(b * xs, taps, w.get(prefix + "conv.bias"))
    return linear(c * cv, w[prefix + "out_proj.weight"], w.get(prefix + "out_proj.bias"))


def swiglu_ffn(h, w, prefix):
    """w2((g * sigmoid(g)) * u), g = w1 h, u = w3 h
    (arch/lib/transformer.json5:117-130; src/graph/cpu.rs:378-390)."""
    g = linear(h, w[prefix + "w1.weight"], w.get(prefix + "w1.bias"))
    u = linear(h, w[prefix + "w3.weight"], w.get(prefix + "w3.bias"))
    sig = 1.0 / (1.0 + torch.exp(-g))
    return linear((g * sig) * u, w[prefix + "w2.weight"], w.get(prefix + "w2.bias"))


def forward(cfg: dict, weights: dict, ids, dtype=torch.float64, rows=None, device="cpu") -> torch.Tensor:
    """Logits [n, vocab] of one whole sequence at positions 0..n-1
    (layer loop: arch/families/lfm2.json5:73-92).  A layer is a conv layer
    when the checkpoint has its ``conv.in_proj.weight``
    (arch/families/lfm2.json5:78-80).  ``rows``: only these positions pass
    through the final norm and the head (the reference's ``head: 'last'``,
    arch/lib/transformer.json5:190, for any rows).  ``device``: where torch
    computes; the formulas are the same anywhere."""
    sizes = resolve_sizes(cfg)
    w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}
    ids = torch.as_tensor(ids, dtype=torch.long, device=device)
    positions = torch.arange(len(ids), device=device)
    x = w["model.embed_tokens.weight"][ids]
    for i in range(sizes["layers"]):
        p = f"model.layers.{i}."
        h = rms_norm(x, w[p + "operator_norm.weight"], sizes["eps"])
        if p + "conv.in_proj.weight" in w:
            a = short_conv_mixer(h, w, p + "conv.", sizes)
        else:
            a = attention_mixer(h, w, p + "self_attn.", sizes, positions)
        x = x + a
        h = rms_norm(x, w[p + "ffn_norm.weight"], sizes["eps"])
        x = x + swiglu_ffn(h, w, p + "feed_forward.")
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long, device=device)]
    z = rms_norm(x, w["model.embedding_norm.weight"], sizes["eps"])
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(z, head)


def greedy(cfg, weights, prompt, n_new, dtype=torch.float64):
    """Greedy continuation: index of the first maximum (src/runtime/lm.rs:1043-1057)."""
    ids = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, weights, ids, dtype)[-1]
        ids.append(int(torch.argmax(logits)))
    return ids[len(prompt):]


# ----------------------------------------------------------------------------
# sampling (src/runtime/lm.rs:1062-1235)
# ----------------------------------------------------------------------------

def penalized(logits, recent, penalty, greedy):
    """The logits after the repetition penalty (float32 arithmetic as the reference's).  A token
    that occurs c times among ``recent`` (the latest 64 tokens count): c times v / penalty if
    v > 0 else v * penalty; the greedy rule then subtracts 1.5 * c (src/runtime/lm.rs:1086-1101),
    the sampling rule subtracts 1.5 after each of the c steps (src/runtime/lm.rs:1171-1190).
    A penalty of 1 or less, or no recent tokens, changes nothing (src/runtime/lm.rs:1074, 1163)."""
    out = np.array(logits, dtype=np.float32, copy=True)
    recent = [int(t) for t in recent][-64:]
    if not penalty > 1.0 or not recent:
        return out
    pen = np.float32(penalty)
    for tok in sorted(set(recent)):
        if not 0 <= tok < len(out):
            continue
        c = recent.count(tok)
        v = out[tok]
        for _ in range(c):
            v = np.float32(v / pen) if v > 0 else np.float32(v * pen)
            if not greedy:
                v = np.float32(v - np.float32(1.5))
        if greedy:
            v = np.float32(v - np.float32(c) * np.float32(1.5))
        out[tok] = v
    return out


def greedy_penalized(cfg, weights, prompt, n_new, penalty, dtype=torch.float64):
    """Greedy continuation under a repetition penalty over the latest 64 tokens of prompt +
    generated (src/scheduler/mod.rs:34-36, 79; src/runtime/lm.rs:1073-1108)."""
    ids = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, weights, ids, dtype)[-1].to(torch.float32).numpy()
        ids.append(int(np.argmax(penalized(logits, ids[-64:], penalty, True))))
    return ids[len(prompt):]


def nucleus_candidates(logits, temperature, top_k, top_p):
    """Top-k by (logit desc, id asc), softmax at the temperature over them,
    shortest prefix whose cumulative probability reaches clamp(top_p, 0.01, 1)
    (src/runtime/lm.rs:1153-1235).  Returns (ids, probs) of the kept prefix,
    probs normalised over the top-k (not over the prefix)."""
    logits = np.asarray(logits, dtype=np.float32)
    k = max(1, min(top_k if top_k > 0 else len(logits), len(logits)))
    order = np.lexsort((np.arange(len(logits)), -logits.astype(np.float64)))[:k]
    vals = logits[order].astype(np.float64) / temperature
    e = np.exp(vals - vals.max())
    probs = e / max(e.sum(), 1e-12)
    thresh = min(max(top_p, 0.01), 1.0)
    cum = np.cumsum(probs)
    cut = int(np.searchsorted(cum, thresh - 1e-12) + 1)
    cut = min(cut, k)
    return order[:cut], probs[:cut]
