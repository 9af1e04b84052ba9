"""The shapes the benchmark itself runs, against an oracle.

A 2,048-token prompt at the LFM2-1.2B widths walks branches that small models
never reach: the CTA-pair product gives every pair several tiles (the phase
bits of its double-buffered accumulator change), the tcgen05 attention kernel
runs 16 key tiles per CTA over 8 kv heads, a product into the residual stream
is deferred whole, and the step walker and the Python wrappers each choose
splits, pairs and kernels from the step's sizes.  Here those products and that
attention launch are compared with float64 restatements, and a two-layer model
(short convolution + attention) with the benchmark's widths is stepped whole,
in portions and token by token: float32 against the plain implementation,
bfloat16 against the float32 engine, the walker against the wrappers bit for
bit.  The reference's rule is that every cutting equals one pass
(MisterTK/gibbs src/runtime/lm.rs:1513-1545).
"""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from helpers import TOL, random_ids, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf16(t):
    d = t.to(torch.bfloat16).to(DEV)
    return d, d.double()


def _rel(got, want):
    got, want = got.double(), want.double()
    return ((got - want).abs().max() / (want.abs().max() + 1e-30)).item()


# --------------------------------------------------------------------------- the products of a 2,048-token step
def test_gate_up_product_with_swiglu_at_2048_tokens():
    """2,048 x 16,384 x 2,048: 8 x 64 tiles of 256 x 256 over 74 CTA pairs, seven tiles a pair."""
    from gibbs_b200 import ops
    from gibbs_b200.parts.linear import interleave_gate_up
    torch.manual_seed(1)
    m, f, k = 2048, 8192, 2048
    a, ar = _bf16(torch.randn(m, k))
    wg, wgr = _bf16(torch.randn(f, k) / math.sqrt(k) * 2)
    wu, wur = _bf16(torch.randn(f, k) / math.sqrt(k) * 2)
    w = interleave_gate_up(wg, wu)
    g, u = ar @ wgr.T, ar @ wur.T
    want = g / (1 + torch.exp(-g)) * u
    out = torch.full((m, f), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(a, w, None, out, swiglu=True)
    assert _rel(out, want) < 2e-2
    # every tile, not only the largest value: row-wise relative error
    assert rel_err(out.float().cpu().numpy(), want.cpu().numpy()) < 1e-2
    assert int(ops.device_status(DEV).item()) == 0


@pytest.mark.parametrize("m,n,k", [(2048, 6144, 2048), (8192, 2048, 2048), (2048, 3072, 2048), (2048, 4608, 1536)])
def test_plain_products_of_a_prompt(m, n, k):
    """in_proj / qkv sized products on CTA pairs with more tiles than pairs, bf16 and f32 stores."""
    from gibbs_b200 import ops
    torch.manual_seed(m + n)
    a, ar = _bf16(torch.randn(m, k))
    w, wr = _bf16(torch.randn(n, k) / math.sqrt(k))
    bias = torch.randn(n, device=DEV)
    exact = ar @ wr.T
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.linear_tc(a, w, None, out)
    assert _rel(out, exact) < 2e-5
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(a, w, bias, out)
    assert _rel(out, exact + bias.double()) < 2e-2
    assert int(ops.device_status(DEV).item()) == 0


@pytest.mark.parametrize("m,n,k", [(2048, 2048, 8192), (2048, 2048, 2048), (2048, 1536, 6912), (512, 2048, 8192)])
def test_product_into_the_residual_stream_deferred_whole_then_normed(m, n, k):
    """down / out_proj of a prompt: from 256 rows on an unsplit product only stores its result
    and the norm that reads the stream next adds it; the stream and the normed rows are checked.
    At 512 rows the same product splits K instead and leaves several partial tiles."""
    from gibbs_b200 import ops
    torch.manual_seed(n + k)
    eps = 1e-5
    a, ar = _bf16(torch.randn(m, k))
    w, wr = _bf16(torch.randn(n, k) / math.sqrt(k))
    gain = (1 + 0.1 * torch.randn(n)).to(DEV)
    x0 = torch.randn(m, n, device=DEV)
    x = x0.clone()
    ws = ops.linear_tc(a, w, None, x, accumulate=True, defer=True)
    assert ws is not x and ws.shape[1:] == (m, n)
    assert torch.equal(x, x0)                                   # nothing was added yet
    want_x = x0.double() + ar @ wr.T
    want_h = want_x / torch.sqrt((want_x ** 2).mean(-1, keepdim=True) + eps) * gain.double()
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x, gain, eps, out, None, pending=(ws, None))
    assert _rel(x, want_x) < 2e-5
    assert _rel(out, want_h) < 2e-2
    # and the read-modify-write epilogue (no deferral) gives the same stream
    x2 = x0.clone()
    ops.linear_tc(a, w, None, x2, accumulate=True)
    assert _rel(x2, want_x) < 2e-5
    assert int(ops.device_status(DEV).item()) == 0


# --------------------------------------------------------------------------- the attention launch of a 2,048-token step
def _dense_causal(q, k, v, heads, kvh, hd, start, scale):
    """float64 attention of a portion that starts at position ``start``: q [n, heads*hd],
    k, v [start + n, kvh, hd]."""
    n = q.shape[0]
    q = q.double().reshape(n, heads, hd).transpose(0, 1)                       # [heads, n, hd]
    rep = heads // kvh
    kk = k.double().transpose(0, 1).repeat_interleave(rep, 0)                  # [heads, L, hd]
    vv = v.double().transpose(0, 1).repeat_interleave(rep, 0)
    s = torch.einsum("hnd,hld->hnl", q, kk) * scale
    pos = torch.arange(start, start + n, device=q.device)
    keys = torch.arange(k.shape[0], device=q.device)
    s = s.masked_fill(keys[None, None, :] > pos[None, :, None], float("-inf"))
    return torch.einsum("hnl,hld->hnd", torch.softmax(s, -1), vv).transpose(0, 1).reshape(n, heads * hd)


class _Hints:
    def __init__(self, before, q_lens):
        t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
        self.n_requests = len(q_lens)
        self.q_start = t([int(v) for v in np.cumsum([0] + q_lens[:-1])])
        self.q_len, self.start_pos = t(q_lens), t(before)
        self.max_q_len = max(q_lens)
        self.max_ctx_len = max(a + b for a, b in zip(before, q_lens))


@pytest.mark.parametrize("heads,kvh,start,n,hd", [(32, 8, 0, 2048, 64), (32, 8, 2048, 2048, 64), (24, 8, 100, 2000, 64),
                                                  (16, 4, 0, 4096, 128), (16, 4, 1000, 1100, 128)])
def test_prompt_attention_at_2048_tokens(heads, kvh, start, n, hd):
    """The tcgen05 kernel with 16 (and 32) key tiles a CTA over 8 kv heads, pages in a random
    order; one key far back is made dominant for the last token of the portion.  Head size 128:
    a launch of more than 444 CTAs, which takes key tiles of 64, and one below, with tiles of 128."""
    from gibbs_b200 import ops
    torch.manual_seed(heads + start)
    ps = 16
    total = start + n
    nb = -(-total // ps)
    perm = torch.randperm(nb + 5)[:nb]
    k = (torch.randn(total, kvh, hd) * 0.5).to(torch.bfloat16)
    v = torch.randn(total, kvh, hd).to(torch.bfloat16)
    q = (torch.randn(n, heads * hd) * 0.5).to(torch.bfloat16)
    far = 77
    q[-1, :hd] = 3.0
    k[far, 0] = 3.0
    v[far, 0] = 50.0
    kp = torch.zeros(nb + 5, kvh, ps, hd, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    pad = nb * ps - total
    kk = torch.cat([k, torch.zeros(pad, kvh, hd, dtype=torch.bfloat16)]).reshape(nb, ps, kvh, hd).transpose(1, 2)
    vv = torch.cat([v, torch.zeros(pad, kvh, hd, dtype=torch.bfloat16)]).reshape(nb, ps, kvh, hd).transpose(1, 2)
    kp[perm], vp[perm] = kk, vv
    scale = 1.0 / math.sqrt(hd)
    want = _dense_causal(q.to(DEV), k.to(DEV), v.to(DEV), heads, kvh, hd, start, scale)
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((n, heads * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    before = ops.launch_count()
    ops.paged_attention(q.to(DEV), heads, kvh, hd, kp.to(DEV), vp.to(DEV), perm.to(torch.int32)[None, :].to(DEV),
                        t([0] * n), t(list(range(start, total))), scale, 0, out, status, hints=_Hints([start], [n]))
    assert ops.launch_count() - before == 1
    assert _rel(out, want) < 2e-2
    assert rel_err(out.float().cpu().numpy(), want.cpu().numpy()) < 2e-2
    assert out[-1, :hd].float().min().item() > 45.0            # the far key was seen
    assert int(status.item()) == 0


# --------------------------------------------------------------------------- two layers at the benchmark's widths
WIDTHS = {
    "1.2B": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288, ffn=8192),
    "700M": dict(hidden_size=1536, num_attention_heads=24, num_key_value_heads=8, intermediate_size=10240, ffn=6912),
}
PROMPT, TAIL = 2048, 32
PORTIONS = (512, 1024, 510, 2)
WANT = [0, 1, 511, 512, 1535, 1536, 2045, 2046, 2047]


def _wide_folder(tmp_path, name):
    from gibbs_b200 import Lfm2Config, write_random_model
    sizes = dict(WIDTHS[name])
    ffn = sizes.pop("ffn")
    raw = dict(architectures=["Lfm2ForCausalLM"], num_hidden_layers=2, head_dim=64, vocab_size=65536,
               block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256, conv_L_cache=3,
               layer_types=["conv", "full_attention"], rope_theta=1000000.0, norm_eps=1e-5, tie_embedding=True,
               max_position_embeddings=4096, **sizes)
    cfg = Lfm2Config.from_dict(raw)
    assert cfg.ffn_dim == ffn
    return write_random_model(tmp_path / name, cfg, seed=2, dtype=torch.bfloat16, gain_jitter=0.1)


def _run(eng, ids, portions):
    """Prompt in the given portions, then the tail token by token; logits at WANT and at every
    tail position, [len(WANT) + TAIL, vocab]."""
    from gibbs_b200 import StepEntry
    eng.open("r")
    rows, pos = [], 0
    for n in portions:
        want = [r - pos for r in WANT if pos <= r < pos + n]
        out = eng.step([StepEntry("r", ids[pos:pos + n], want)])
        if want:
            rows.append(out.clone())
        pos += n
    assert pos == PROMPT
    for t in range(TAIL):
        rows.append(eng.step([StepEntry("r", [ids[PROMPT + t]], [0])]).clone())
    eng.close("r")
    eng.check_status()
    eng.cache.check()
    return torch.cat(rows).cpu().numpy()


@pytest.mark.parametrize("name", ["1.2B", "700M"])
def test_two_layers_at_benchmark_widths_whole_cut_and_decoded(tmp_path, name):
    from gibbs_b200 import Engine, load_model
    folder = _wide_folder(tmp_path, name)
    ids = random_ids(8, PROMPT + TAIL, 65536)
    cfg, w = plain.load_folder(folder)
    rows = WANT + list(range(PROMPT, PROMPT + TAIL))
    want = plain.forward(cfg, w, ids, rows=rows, device=DEV).cpu().numpy()
    del w
    n_pages = (PROMPT + TAIL) // 16 + 2
    got = {}
    for dtype in ("float32", "bfloat16"):
        model = load_model(folder, dtype=dtype)
        for use_plan in ((True, False) if dtype == "bfloat16" else (True,)):
            eng = Engine(model, n_pages=n_pages, page_size=16, max_requests=2, max_step_tokens=PROMPT,
                         use_plan=use_plan)
            assert (eng.plan is not None) == use_plan, eng.plan_refusal
            got[dtype, use_plan, "whole"] = _run(eng, ids, (PROMPT,))
            got[dtype, use_plan, "cut"] = _run(eng, ids, PORTIONS)
            del eng
        del model
        torch.cuda.empty_cache()
    for how in ("whole", "cut"):
        f32, b16 = got["float32", True, how], got["bfloat16", True, how]
        # float32 against the float64 plain implementation; the sums are 2,048 to 8,192 terms long
        assert rel_err(f32, want) < 2e-5, (name, how, rel_err(f32, want))
        assert rel_err(b16, f32) < TOL["bfloat16"], (name, how, rel_err(b16, f32))
        assert rel_err(b16, want) < TOL["bfloat16"]
        # the walker and the Python wrappers launch the same kernels with the same arguments
        assert np.array_equal(b16, got["bfloat16", False, how]), (name, how)


@pytest.mark.parametrize("name", ["1.2B", "700M"])
def test_random_mixed_batches_at_benchmark_widths(tmp_path, name):
    """Up to four live requests of 13 to 712 tokens, portions of some beside decoded tokens of others,
    in a pool so small that pages are used again, with and without decode graphs and the step plan,
    step after step without a host wait: the bfloat16 engine's logits at the last place of every
    portion against the float32 engine running each request whole."""
    from gibbs_b200 import Engine, StepEntry, load_model
    from helpers import trace_mixed
    folder = _wide_folder(tmp_path, name)
    m32, m16 = load_model(folder, dtype="float32"), load_model(folder, dtype="bfloat16")
    for seed in range(1, 7):
        rng = np.random.default_rng(seed)
        lens = [int(rng.choice([1, 2, 33, 64, 100, 129, 255, 256, 257, 400, 513, 700])) + 12
                for _ in range(int(rng.integers(3, 7)))]
        reqs = {f"s{seed}r{i}": random_ids(seed * 100 + i, n, 65536) for i, n in enumerate(lens)}
        cap = max(-(-max(lens) // 64) * 64 + 64, int(rng.choice([512, 896, 1408])))
        steps = trace_mixed(reqs, capacity_tokens=cap, max_live=4, seed=seed)
        for s in steps:
            for e in s["entries"]:
                e["want"] = e["want"][-1:]
        eng = Engine(m16, n_pages=cap // 16 + 4, page_size=16, max_requests=4, max_step_tokens=2048,
                     use_graphs=bool(seed & 1), use_plan=seed != 4)
        got = {}
        for s in steps:
            for ent in s["entries"]:
                if not eng.is_live(ent["id"]):
                    eng.open(ent["id"])
            bases = {ent["id"]: eng.length(ent["id"]) for ent in s["entries"]}
            logits = eng.step([StepEntry(ent["id"], ent["tokens"], ent["want"]) for ent in s["entries"]])
            if logits is not None:
                logits, row = logits.clone(), 0
                for ent in s["entries"]:
                    for w in ent["want"]:
                        got.setdefault(ent["id"], {})[bases[ent["id"]] + w] = logits[row]
                        row += 1
            for rid in s["end"]:
                eng.close(rid)
        torch.cuda.synchronize()
        eng.check_status()
        eng.cache.check()
        del eng
        ref = Engine(m32, n_pages=max(lens) // 16 + 4, page_size=16, max_requests=1, max_step_tokens=2048)
        for rid, ids in reqs.items():
            places = sorted(got[rid])
            ref.open(rid)
            want = ref.step([StepEntry(rid, ids, places)]).double()
            ref.close(rid)
            have = torch.stack([got[rid][p] for p in places]).double()
            err = (have - want).norm(dim=-1) / (want.norm(dim=-1) + 1e-30)
            assert float(err.max()) < TOL["bfloat16"], \
                f"seed {seed}: request {rid} of {len(ids)}, place {places[int(err.argmax())]}: rel err {float(err.max()):.3g}"
        del ref


# --------------------------------------------------------------------------- the whole benchmark model and its 32-bit twin
def test_full_size_model_in_bfloat16_against_its_float32_twin():
    """All 16 layers of the LFM2-1.2B shape with random bfloat16 weights: the bfloat16 engine against
    the float32 engine on the same (rounded) weights, which is its exact twin: a 512-token prompt
    whole, the same in portions, and 32 tokens decoded one by one."""
    from gibbs_b200 import Engine, Lfm2Config, StepEntry
    from gibbs_b200.parts import build_model
    from gibbs_b200.weights import TensorDict, random_tensors
    raw = dict(architectures=["Lfm2ForCausalLM"], hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, vocab_size=65536, intermediate_size=12288,
               block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256, conv_L_cache=3,
               full_attn_idxs=[2, 5, 8, 10, 12, 14], rope_theta=1000000.0, norm_eps=1e-5, tie_embedding=True,
               max_position_embeddings=4096)
    cfg = Lfm2Config.from_dict(raw)
    plan = cfg.plan()
    tensors = TensorDict(dict(random_tensors(plan, 2, torch.bfloat16, gain_jitter=0.1)))
    prompt, tail = 512, 32
    ids = random_ids(21, prompt + tail, 65536)
    want_rows = [0, 255, 256, 511]

    def run(eng, portions):
        eng.open("r")
        rows, pos = [], 0
        for n in portions:
            want = [r - pos for r in want_rows if pos <= r < pos + n]
            out = eng.step([StepEntry("r", ids[pos:pos + n], want)])
            if want:
                rows.append(out.clone())
            pos += n
        for t in range(tail):
            rows.append(eng.step([StepEntry("r", [ids[prompt + t]], [0])]).clone())
        eng.close("r")
        eng.check_status()
        return torch.cat(rows).cpu().numpy()

    got = {}
    for dtype in (torch.float32, torch.bfloat16):
        model = build_model(plan, tensors, dtype, DEV)
        eng = Engine(model, n_pages=(prompt + tail) // 16 + 2, page_size=16, max_requests=1, max_step_tokens=prompt)
        got[dtype, "whole"] = run(eng, (prompt,))
        got[dtype, "cut"] = run(eng, (200, 2, 310))
        del eng, model
        torch.cuda.empty_cache()
    f32, b16 = got[torch.float32, "whole"], got[torch.bfloat16, "whole"]
    assert rel_err(got[torch.float32, "cut"], f32) < 2e-5
    # The bound of the tiny models (4 and 6 layers) holds for their depth: every layer rounds its
    # activations to bfloat16 anew, independent errors add in quadrature, so 16 layers carry about
    # sqrt(16 / 4) = 2 times the error of 4 (measured: 2.3e-2 against 5e-3 to 7e-3).
    bound = TOL["bfloat16"] * math.sqrt(16 / 4)
    assert rel_err(b16, f32) < bound, rel_err(b16, f32)
    assert rel_err(got[torch.bfloat16, "cut"], f32) < bound
    # greedy choices agree wherever the 32-bit logits are not within rounding of a tie
    for row32, row16 in zip(f32, b16):
        top = int(np.argmax(row16))
        assert row32.max() - row32[top] <= 0.02 * (row32.max() - row32.min())
