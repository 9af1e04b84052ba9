"""The plain implementation itself (no GPU): anchored on the reference's frozen
LFM2 golden logits, plus properties of each part."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from helpers import TINY, make_folder, random_ids

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import make_anchor  # noqa: E402


@pytest.fixture(scope="module")
def fixture_folder(tmp_path_factory):
    return make_anchor.write_fixture(tmp_path_factory.mktemp("anchor"))


def test_plain_reproduces_the_reference_golden(fixture_folder):
    cfg, w = plain.load_folder(fixture_folder)
    ref = make_anchor.golden()
    for name, ids in make_anchor.golden_cases():
        got = plain.forward(cfg, w, ids)[-1].numpy()
        want = np.array(ref["f32"][name])
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        cos = got @ want / np.linalg.norm(got) / np.linalg.norm(want)
        # the reference's own bound is rel < 1e-3, cos > 0.9999 (tests/golden/util.rs:257-260);
        # its numbers are float32, so agreement stops near 1e-6
        assert rel < 5e-6 and cos > 0.999999, (name, rel)
    assert plain.greedy(cfg, w, make_anchor.PROMPT6, 8) == ref["ids"]["greedy8"]


def test_committed_anchor_report_is_current(fixture_folder):
    report = json.loads((Path(make_anchor.HERE) / "anchor_report.json").read_text())
    assert report["greedy8"]["plain"] == report["greedy8"]["reference"]
    assert all(c["rel_l2"] < 5e-6 for c in report["cases"].values())


def test_conv_tap_order_and_bias():
    # an impulse at t=2 on one channel comes out as taps[K-1], taps[K-2], ... at t=2, 3, ...
    bx = torch.zeros(6, 2, dtype=torch.float64)
    bx[2, 1] = 1.0
    taps = torch.tensor([[0.0, 0.0, 0.0], [10.0, 20.0, 30.0]], dtype=torch.float64)
    out = plain.causal_conv1d(bx, taps)
    assert out[:, 1].tolist() == [0, 0, 30.0, 20.0, 10.0, 0] and float(out[:, 0].abs().sum()) == 0
    assert plain.causal_conv1d(bx, taps, torch.tensor([1.0, 2.0], dtype=torch.float64))[0].tolist() == [1.0, 2.0]


def test_rope_is_a_rotation_of_half_split_pairs():
    x = torch.randn(5, 3, 8, dtype=torch.float64)
    inv = plain.rope_inv_freq(8, 10000.0, torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 4000])
    y = plain.rope_half_split(x, pos, inv)
    assert torch.allclose(y[0], x[0])                                   # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    a = float(pos[2]) * float(inv[1])
    assert abs(float(y[2, 0, 1]) - (float(x[2, 0, 1]) * np.cos(a) - float(x[2, 0, 5]) * np.sin(a))) < 1e-6
    assert abs(float(inv[1]) - np.float32(1.0) / np.float32(10000.0) ** np.float32(0.25)) < 1e-9


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8, dtype=torch.float64), torch.randn(6, 2, 8, dtype=torch.float64), \
        torch.randn(6, 2, 8, dtype=torch.float64)
    o = plain.causal_attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0
    assert torch.allclose(plain.causal_attention(q, k2, v2, 0.3)[:4], o[:4])      # the future is not seen
    assert torch.allclose(o[0, 1], v[0, 0]) and torch.allclose(o[0, 2], v[0, 1])   # heads 0,1 -> kv 0; 2,3 -> kv 1
    ow = plain.causal_attention(q, k, v, 0.3, window=2)
    k3 = k.clone()
    k3[:3] = 5.0
    assert torch.allclose(plain.causal_attention(q, k3, v, 0.3, window=2)[4:], ow[4:])   # keys 0..2 are outside


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    g = torch.tensor([2.0, 0.5], dtype=torch.float64)
    want = x / np.sqrt(12.5 + 1e-5) * g
    assert torch.allclose(plain.rms_norm(x, g, 1e-5), want)
    w = {"p.w1.weight": torch.eye(2, dtype=torch.float64), "p.w3.weight": 2 * torch.eye(2, dtype=torch.float64),
         "p.w2.weight": torch.eye(2, dtype=torch.float64)}
    got = plain.swiglu_ffn(x, w, "p.")
    assert torch.allclose(got, (x / (1 + torch.exp(-x))) * (2 * x))


def test_forward_is_prefix_stable_and_uses_every_option(tmp_path):
    for name in ("A", "B"):
        folder = make_folder(tmp_path, name)
        cfg, w = plain.load_folder(folder)
        ids = random_ids(3, 30, TINY[name][0]["vocab_size"])
        full = plain.forward(cfg, w, ids)
        assert torch.allclose(plain.forward(cfg, w, ids[:11]), full[:11], atol=1e-12)
        # every tensor of the checkpoint changes the logits
        for key in w:
            w2 = dict(w)
            w2[key] = w[key] + 0.05
            assert not torch.allclose(plain.forward(cfg, w2, ids), full, atol=1e-9), key
    assert plain.resolve_sizes(TINY["B"][0])["inter"] == 256


def test_nucleus_candidates():
    logits = np.array([0.1, 3.0, 3.0, 2.0, -1.0, 2.5], dtype=np.float32)
    ids, probs = plain.nucleus_candidates(logits, 1.0, 4, 1.0)
    assert ids.tolist() == [1, 2, 5, 3] and abs(probs.sum() - 1) < 1e-9       # ties: lower id first
    ids, probs = plain.nucleus_candidates(logits, 1.0, 4, 0.5)
    assert ids.tolist() == [1, 2]
    ids, _ = plain.nucleus_candidates(logits, 0.5, 64, 0.0)                    # top_p clamps to 0.01
    assert ids.tolist() == [1]
