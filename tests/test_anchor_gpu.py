"""The engine against the reference's own numbers, and at the benchmark's layer sizes.

1. The reference's frozen LFM2 fixture (3 layers, head size 8, vocabulary 256; weights from its
   SplitMix64 stream) runs through the engine; the logits are compared with the golden file the
   reference ships (tests/golden/ref_lfm2_golden.json), in the way the reference produced them:
   a prompt in one pass, then forced tokens one by one, and greedy decoding.
2. Two layers with the LFM2-1.2B widths (hidden 2048, 32/8 heads of 64, feed-forward 8192,
   vocabulary 65536): float32 against the plain implementation, bfloat16 against the float32
   engine, whole and cut, so that every kernel runs at the sizes the benchmark uses.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import make_anchor  # noqa: E402
from helpers import TOL, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_reproduces_the_reference_golden(tmp_path, dtype):
    from gibbs_b200 import Generator, SamplingParams, StepEntry
    folder = make_anchor.write_fixture(tmp_path / "fixture")
    ref = make_anchor.golden()
    gen = Generator(folder, dtype=dtype, ctx=128, page_size=16, n_pages=16, max_running=2)
    eng = gen.engine
    # the reference's own bound is rel < 1e-3 and cos > 0.9999 (tests/golden/util.rs:257-260); its
    # golden values are float32, so the float32 engine agrees to rounding
    tol = 5e-6 if dtype == "float32" else TOL["bfloat16"]

    def check(name, got):
        want = np.array(ref["f32"][name])
        assert rel_err(got[None, :], want[None, :]) < tol, name
        if dtype == "float32":
            assert got @ want / np.linalg.norm(got) / np.linalg.norm(want) > 0.9999

    eng.open("p6")
    check("prefill6", eng.step([StepEntry("p6", make_anchor.PROMPT6, [5])])[0].cpu().numpy().astype(np.float64))
    for i, tok in enumerate(make_anchor.FORCED):
        check(f"decode{i}", eng.step([StepEntry("p6", [tok], [0])])[0].cpu().numpy().astype(np.float64))
    eng.open("p20")      # beside the live first request
    check("prefill20", eng.step([StepEntry("p20", make_anchor.PROMPT20, [19])])[0].cpu().numpy().astype(np.float64))
    eng.close("p6"), eng.close("p20")
    if dtype == "float32":
        out = gen.generate([make_anchor.PROMPT6], SamplingParams(temperature=0.0, max_new_tokens=8),
                           stop_at_eos=False)[0]
        assert out == ref["ids"]["greedy8"]


def test_benchmark_layer_sizes_float32_and_bfloat16(tmp_path):
    from gibbs_b200 import Engine, Lfm2Config, StepEntry, load_model, write_random_model
    raw = dict(architectures=["Lfm2ForCausalLM"], hidden_size=2048, num_hidden_layers=2, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, vocab_size=65536, intermediate_size=12288,
               block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256, conv_L_cache=3,
               layer_types=["conv", "full_attention"], rope_theta=1000000.0, norm_eps=1e-5, tie_embedding=True,
               max_position_embeddings=512)
    cfg = Lfm2Config.from_dict(raw)
    assert cfg.ffn_dim == 8192
    folder = write_random_model(tmp_path / "wide", cfg, seed=2, dtype=torch.bfloat16, gain_jitter=0.1)
    ids = random_ids(8, 150, 65536)
    want_rows = [0, 1, 63, 64, 65, 127, 149]
    want = plain_logits(folder, ids)[want_rows]
    logits = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(load_model(folder, dtype=dtype), n_pages=24, page_size=16, max_requests=2, max_step_tokens=256)
        eng.open("w")
        whole = eng.step([StepEntry("w", ids, want_rows)]).cpu().numpy()
        eng.close("w")
        eng.open("c")
        got, pos = {}, 0
        for n in (64, 2, 61, 1, 1, 1, 20):                       # a page edge, two tokens, single tokens
            rows = [r - pos for r in want_rows if pos <= r < pos + n]
            out = eng.step([StepEntry("c", ids[pos:pos + n], rows)])
            for k, r in enumerate(rows):
                got[pos + r] = out[k].cpu().numpy()
            pos += n
        eng.close("c")
        eng.check_status()
        cut = np.stack([got[r] for r in want_rows])
        logits[dtype] = whole
        # float32: against the float64 plain implementation; the sums are 2048 to 8192 terms long
        tol = 2e-5 if dtype == "float32" else TOL["bfloat16"]
        assert rel_err(whole, want) < tol, (dtype, rel_err(whole, want))
        assert rel_err(cut, want) < tol, (dtype, rel_err(cut, want))
    assert rel_err(logits["bfloat16"], logits["float32"]) < TOL["bfloat16"]
