"""Generation through the public entry point and the command line."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from helpers import TINY, TOL, make_folder, plain_logits, random_ids, rel_err

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _gen(folder, dtype, **kw):
    from gibbs_b200 import Generator
    args = dict(dtype=dtype, device="cuda:0", ctx=512, page_size=16, n_pages=64, max_running=4)
    args.update(kw)
    return Generator(folder, **args)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_float32_equals_plain(tmp_path, name):
    from gibbs_b200 import SamplingParams
    folder = make_folder(tmp_path, name, std=0.05)
    cfg, w = plain.load_folder(folder)
    vocab = TINY[name][0]["vocab_size"]
    prompts = [random_ids(5, 7, vocab), random_ids(6, 13, vocab), [3]]
    gen = _gen(folder, "float32")
    outs = gen.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8), stop_at_eos=False)
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(cfg, w, p, 8)


def test_greedy_generation_with_a_repetition_penalty_equals_plain(tmp_path):
    """The penalty sees the latest 64 tokens of prompt and generated text; with a strong one the
    continuation differs from the plain greedy one, and equals the plain rule's token by token.
    A request without a penalty in the same batch is not touched."""
    from gibbs_b200 import SamplingParams
    folder = make_folder(tmp_path, "A", std=0.05)
    cfg, w = plain.load_folder(folder)
    prompts = [random_ids(5, 70, 512), random_ids(6, 9, 512)]
    gen = _gen(folder, "float32")
    pen = SamplingParams(temperature=0.0, max_new_tokens=24, repetition_penalty=1.8)
    outs = gen.generate(prompts, [pen, SamplingParams(temperature=0.0, max_new_tokens=24)], stop_at_eos=False)
    assert outs[0] == plain.greedy_penalized(cfg, w, prompts[0], 24, 1.8)
    assert outs[1] == plain.greedy(cfg, w, prompts[1], 24)
    assert outs[0] != plain.greedy(cfg, w, prompts[0], 24)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_follows_the_plain_logits(tmp_path, dtype):
    """300 tokens decoded one by one (through CUDA graphs in steady state): every
    token must be the plain model's choice given the same history; in bfloat16
    a token may differ only where the plain logits are within rounding."""
    from gibbs_b200 import SamplingParams
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, "A", stored=stored, std=0.05)
    prompt = random_ids(9, 20, 512)
    gen = _gen(folder, dtype)
    out = gen.generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=300), stop_at_eos=False)[0]
    assert len(out) == 300
    logits = plain_logits(folder, prompt + out)              # teacher forced on the engine's own tokens
    for t, tok in enumerate(out):
        row = logits[len(prompt) + t - 1]
        if dtype == "float32":
            assert tok == int(np.argmax(row)), t
        else:
            assert row.max() - row[tok] <= 0.02 * (row.max() - row.min()), t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tmp_path, dtype):
    from gibbs_b200 import StepEntry
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, "B", stored=stored)
    ids = random_ids(1, 6, 1000)
    want = plain_logits(folder, ids)
    eng = _gen(folder, dtype).engine
    for cut in ([1, 1, 1, 1, 1, 1], [1, 2, 3], [2, 1, 3], [3, 3]):
        eng.open("s")
        got, pos = [], 0
        for n in cut:
            got.append(eng.step([StepEntry("s", ids[pos:pos + n], list(range(n)))]).cpu().numpy())
            pos += n
        eng.close("s")
        assert rel_err(np.concatenate(got), want) < TOL[dtype], cut


def test_temperature_sampling_is_seeded_and_stays_in_the_top_k(tmp_path):
    from gibbs_b200 import SamplingParams
    folder = make_folder(tmp_path, "A", std=0.08)
    prompt = random_ids(2, 10, 512)
    gen = _gen(folder, "float32")
    p = SamplingParams(temperature=0.9, top_k=5, top_p=0.95, max_new_tokens=24, seed=123)
    a = gen.generate([prompt], p, stop_at_eos=False)[0]
    b = gen.generate([prompt], p, stop_at_eos=False)[0]
    c = gen.generate([prompt], SamplingParams(temperature=0.9, top_k=5, top_p=0.95, max_new_tokens=24, seed=124),
                     stop_at_eos=False)[0]
    assert a == b and a != c
    logits = plain_logits(folder, prompt + a)
    for t, tok in enumerate(a):
        row = logits[len(prompt) + t - 1]
        assert tok in np.argsort(-row)[:5]
    # same seed, other batch composition: a request's draws do not depend on its neighbours
    d = gen.generate([random_ids(3, 4, 512), prompt], [SamplingParams(max_new_tokens=5), p], stop_at_eos=False)[1]
    assert d == a


def test_scheduler_preempts_and_recomputes_on_the_gpu(tmp_path):
    """A pool too small for both requests at full length: the one admitted last
    gives way and is recomputed; tokens equal an unconstrained run."""
    from gibbs_b200 import SamplingParams
    folder = make_folder(tmp_path, "B", std=0.05)
    prompts = [random_ids(11, 30, 1000), random_ids(12, 28, 1000)]
    p = SamplingParams(temperature=0.0, max_new_tokens=40)
    roomy = _gen(folder, "float32", n_pages=64).generate(prompts, p, stop_at_eos=False)
    gen = _gen(folder, "float32", n_pages=7, page_size=16, max_running=2)     # 112 positions for 138
    sched = gen.scheduler(stop_at_eos=False)
    ids = [sched.submit(q, p) for q in prompts]
    preempted = []
    while sched.has_work():
        preempted += sched.step().preempted
    assert preempted and [sched.sequences[i].output for i in ids] == roomy
    assert gen.engine.cache.free_pages() == [7]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_feedback_emits_the_tokens_of_the_plain_loop(tmp_path, dtype):
    """Decode steps launched on the ids the device picked, one step before the host reads
    them, against the loop that reads every id first: the same tokens and finish reasons,
    with greedy and seeded temperature requests, ends by length at different steps and (in
    32-bit, where a changed batch cannot move a choice) an end on a stop id."""
    from gibbs_b200 import SamplingParams
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, "B", stored=stored, std=0.05)
    gen = _gen(folder, dtype)
    prompts = [random_ids(21, 33, 1000), random_ids(22, 5, 1000), random_ids(23, 18, 1000), [7]]
    free = gen.generate([prompts[3]], SamplingParams(temperature=0.0, max_new_tokens=31), stop_at_eos=False)[0]
    stop = (free[12],) if dtype == "float32" else ()
    params = [SamplingParams(temperature=0.0, max_new_tokens=40),
              SamplingParams(temperature=0.8, top_k=8, top_p=0.9, seed=5, max_new_tokens=25),
              SamplingParams(temperature=0.0, max_new_tokens=3),
              SamplingParams(temperature=0.0, max_new_tokens=31, stop_ids=stop)]
    got = []
    for overlap in (False, True):
        sched = gen.scheduler(stop_at_eos=False, overlap=overlap)
        ids = [sched.submit(p, q) for p, q in zip(prompts, params)]
        before = gen.engine.fed_steps
        emitted = {i: [] for i in ids}
        while sched.has_work():
            for i, t in sched.step().emitted:
                emitted[i].append(t)
        fed = gen.engine.fed_steps - before
        assert (fed >= 30) if overlap else (fed == 0)
        assert all(emitted[i] == sched.sequences[i].output for i in ids)
        got.append([(sched.sequences[i].output, sched.sequences[i].finish) for i in ids])
        assert not gen.engine.cache.live
    assert got[0] == got[1]
    if stop:
        assert got[1][3][0] == free[:free.index(stop[0])] and got[1][3][1] == "stop"


@pytest.mark.parametrize("seed", [2, 4, 8])
def test_token_feedback_under_random_traffic_and_page_pressure(tmp_path, seed):
    """Requests arrive while others run, greedy and sampled, with end-of-sequence ids that do end
    some of them and pools so small that requests are preempted: with ids that lag a step the
    scheduler emits what the plain loop emits (32-bit, where a changed batch cannot move a choice)."""
    import random
    from gibbs_b200 import SamplingParams
    folder = make_folder(tmp_path, "B", std=0.05)
    vocab = TINY["B"][0]["vocab_size"]
    rng = random.Random(seed)
    gen = _gen(folder, "float32", ctx=128, n_pages=rng.choice([10, 14, 40]), max_running=rng.choice([2, 4]),
               max_batch_tokens=rng.choice([16, 48]))
    eos = {rng.randrange(vocab) for _ in range(40)}

    def run(overlap):
        r = random.Random(seed + 1000)
        sched = gen.scheduler(stop_at_eos=False, overlap=overlap)
        sched.eos_ids = set(eos)
        ids, before = [], gen.engine.fed_steps
        for step in range(2000):
            if step < 40 and r.random() < 0.35:
                prompt = [r.randrange(vocab) for _ in range(r.randint(1, 50))]
                params = SamplingParams(temperature=r.choice([0.0, 0.9]), top_k=r.choice([1, 5, 50]),
                                        top_p=r.choice([0.5, 1.0]), seed=r.randrange(1 << 30),
                                        max_new_tokens=r.randint(0, 60))
                ids.append(sched.submit(prompt, params))
            if not sched.has_work():
                if step >= 40:
                    break
                continue
            sched.step()
        assert not sched.has_work() and not gen.engine.cache.live
        return [(sched.sequences[i].output, sched.sequences[i].finish) for i in ids], gen.engine.fed_steps - before

    plain_loop, none_fed = run(False)
    lagging, fed = run(True)
    assert none_fed == 0 and fed > 5
    assert plain_loop == lagging


def test_eos_from_config_stops_generation(tmp_path):
    from gibbs_b200 import Lfm2Config, SamplingParams, write_random_model
    raw = dict(TINY["A"][0])
    cfg0, w0 = None, None
    folder = make_folder(tmp_path, "A", std=0.05)
    prompt = random_ids(4, 9, 512)
    free = _gen(folder, "float32").generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=12),
                                            stop_at_eos=False)[0]
    raw["eos_token_id"] = free[4]
    cut = free.index(free[4])
    folder2 = write_random_model(tmp_path / "with_eos", Lfm2Config.from_dict(raw), TINY["A"][1], gain_jitter=0.1,
                                 std=0.05)
    out = _gen(folder2, "float32").generate([prompt], SamplingParams(temperature=0.0, max_new_tokens=12))[0]
    assert out == free[:cut]


def test_command_line(tmp_path):
    folder = make_folder(tmp_path, "A", std=0.05)
    cfg, w = plain.load_folder(folder)
    prompt = [5, 17, 42, 99]
    run = lambda *args: subprocess.run([sys.executable, str(ROOT / "bin" / "gibbs-b200"), *args], text=True,
                                       capture_output=True, timeout=600)
    p = run("--model", str(folder), "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6",
            "--temperature", "0", "--dtype", "float32", "--ctx", "64")
    assert p.returncode == 0, p.stderr[-2000:]
    lines = p.stdout.splitlines()
    out = [int(t) for t in lines[lines.index("Output:") + 1].split(",")]
    assert out == plain.greedy(cfg, w, prompt, 6)
    assert any(l.startswith("Decode: 5 tokens") for l in lines) and any(l.startswith("Roofline:") for l in lines)
    p = run("--model", str(folder), "--probe-top5", "5,17,42", "--dtype", "float32", "--ctx", "64")
    top = json.loads(p.stdout.strip().splitlines()[-1])
    want = plain.forward(cfg, w, [5, 17, 42])[-1].numpy()
    assert top["ids"] == [int(i) for i in np.argsort(-want)[:5]]
    p = run("--model", str(folder), "--arch-dump")
    dump = json.loads(p.stdout)
    assert dump["architecture"] == "Lfm2ForCausalLM" and dump["unconsumed"] == []
    assert dump["config"]["ffn_dim (derived)"] == 192
    (tmp_path / "cfg.json").write_text(json.dumps(TINY["B"][0]))
    p = run("--random", str(tmp_path / "cfg.json"), "--seed", "1", "--save", str(tmp_path / "rnd"), "--dtype",
            "float32")
    assert p.returncode == 0 and (tmp_path / "rnd" / "model.safetensors").exists()
    (tmp_path / "suite.json").write_text(json.dumps({"defaults": {"decode_tokens": 8, "prefill_tokens": 32, "runs": 1},
                                                     "models": [{"id": str(folder)}]}))
    p = run("--model", str(folder), "--bench", str(tmp_path / "suite.json"), "--dtype", "float32")
    assert p.returncode == 0, p.stderr[-2000:]
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    for key in ("decode_tok_s", "prefill_tok_s", "bytes_per_token", "roofline_pct", "wall_ms", "weights_ms"):
        assert key in rec
    shares = rec["kernel_time_shares"]
    assert {"linear:gate_up", "linear:down", "attention", "short_conv", "rmsnorm"} <= set(shares)
    assert abs(sum(shares.values()) - 1.0) < 0.01
    # the peaks that roofline figures relate to come from --peaks, else the built-in figures
    (tmp_path / "peaks.json").write_text(json.dumps({"hbm_gbs": 1234.5, "bf16_tflops": 100.0}))
    p = run("--model", str(folder), "--bench", str(tmp_path / "suite.json"), "--dtype", "float32", "--peaks",
            str(tmp_path / "peaks.json"))
    assert p.returncode == 0 and json.loads(p.stdout.strip().splitlines()[-1])["ceiling_gbps"] == 1234.5
    assert rec["ceiling_gbps"] == 6650.0


@pytest.mark.parametrize("name,ctx", [("A", 64), ("B", 128)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_stops_at_the_contexts_end_and_a_step_past_it_is_refused(tmp_path, name, ctx, dtype):
    """The tiny configurations with the context lengths their descriptions give (64 and 128; the
    other tests give them 512 positions): generation into the context's end finishes with
    ``length`` at exactly ctx tokens (MisterTK/gibbs src/scheduler/mod.rs:1366-1371, 1521-1525),
    the tokens up to there are the plain model's, and a step that would write position ctx is an
    error before anything changes (src/runtime/lm.rs:538-544)."""
    import json as _json
    from gibbs_b200 import Generator, SamplingParams, StepEntry
    from gibbs_b200.engine.scheduler import FinishReason
    from gibbs_b200.engine.step import StepError
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, name, stored=stored, std=0.08)
    cfg_path = Path(folder) / "config.json"
    raw = _json.loads(cfg_path.read_text())
    raw["max_position_embeddings"] = ctx
    cfg_path.write_text(_json.dumps(raw))
    gen = Generator(folder, dtype=dtype, page_size=16, max_running=2)        # ctx from config.json
    assert gen.engine.max_context == ctx
    vocab = TINY[name][0]["vocab_size"]
    prompt = random_ids(3, ctx - 20, vocab)
    sched = gen.scheduler(stop_at_eos=False)
    sid = sched.submit(prompt, SamplingParams(temperature=0.0, max_new_tokens=1000))
    sched.run()
    seq = sched.sequences[sid]
    assert seq.finish == FinishReason.LENGTH and len(prompt) + len(seq.output) == ctx
    logits = plain_logits(folder, prompt + seq.output)
    for t, tok in enumerate(seq.output):
        row = logits[len(prompt) + t - 1]
        if dtype == "float32":
            assert tok == int(np.argmax(row)), t
        else:
            assert row.max() - row[tok] <= 0.02 * (row.max() - row.min()), t
    assert not gen.engine.cache.live
    with pytest.raises(ValueError, match="does not fit the context"):
        sched.submit(random_ids(4, ctx, vocab))
    # the step function itself: the last position is fine, one more is refused and changes nothing
    eng = gen.engine
    eng.open("edge")
    ids = random_ids(5, ctx, vocab)
    out = eng.step([StepEntry("edge", ids, [ctx - 1])])
    want = plain_logits(folder, ids)[-1:]
    assert rel_err(out.cpu().numpy(), want) < TOL[dtype]
    free = eng.cache.free_pages()
    with pytest.raises(StepError, match="the context is"):
        eng.step([StepEntry("edge", [1], [0])])
    assert eng.length("edge") == ctx and eng.cache.free_pages() == free
    eng.close("edge")
    eng.cache.check()


def test_timing_mode_adds_up_the_operations_of_a_step_by_kind(tmp_path):
    """GIBBS_B200_TIMING=1 / Engine(timing=True): the step walker brackets every operation with
    CUDA events and adds the times up per kind (the reference's per-kernel-class table,
    MisterTK/gibbs src/graph/metal.rs:143-148).  The counts are exact, the logits are the
    same bits as without timing."""
    from gibbs_b200 import Engine, StepEntry, load_model
    folder = make_folder(tmp_path, "A", stored=torch.bfloat16, std=0.05)
    model = load_model(folder, dtype="bfloat16")
    ids = random_ids(4, 40, 512)
    outs = []
    for timing in (False, True):
        eng = Engine(model, n_pages=8, page_size=16, max_requests=2, max_step_tokens=64, timing=timing)
        assert eng.plan is not None and eng.use_graphs == (not timing)
        eng.open("t")
        rows = [eng.step([StepEntry("t", ids[:37], [36])]).clone()]
        for t in ids[37:]:
            rows.append(eng.step([StepEntry("t", [t], [0])]).clone())
        outs.append(torch.cat(rows))
        if timing:
            table = eng.timing_table()
        else:
            assert eng.timing_table() == {}
        eng.close("t")
    assert torch.equal(outs[0], outs[1])
    steps, conv_layers, attn_layers = 4, 2, 2                    # tiny A: [conv, attention, conv, attention]
    want = {"embed": steps, "rmsnorm": steps * (2 * 4 + 1), "linear:in_proj": steps * conv_layers,
            "short_conv": steps * conv_layers, "linear:qkv": steps * attn_layers, "qk_rope": steps * attn_layers,
            "attention": steps * attn_layers, "linear:out_proj": steps * 4, "linear:gate_up": steps * 4,
            "linear:down": steps * 4, "linear:lm_head": steps}
    assert {k: n for k, (n, _) in table.items()} == want
    # a norm that the product after it ran itself (decode steps) took no time of its own; everything else did
    assert all(ms > 0 for k, (_, ms) in table.items() if k != "rmsnorm")
    total = sum(ms for _, ms in table.values())
    assert 0 < total < 1000


def test_top_logprobs_through_the_entry_point(tmp_path):
    """A request that asks for top_logprobs gets a report per token whose chosen id is the emitted
    token and whose numbers agree with the plain logits of the same history."""
    from gibbs_b200 import SamplingParams
    folder = make_folder(tmp_path, "A", std=0.08)
    gen = _gen(folder, "float32")
    prompt = random_ids(12, 9, 512)
    sched = gen.scheduler(stop_at_eos=False)
    sid = sched.submit(prompt, SamplingParams(temperature=0.0, max_new_tokens=5, top_logprobs=4))
    sched.run()
    seq = sched.sequences[sid]
    assert len(seq.logprobs) == len(seq.output) == 5
    logits = plain_logits(folder, prompt + seq.output)
    for t, (tok, info) in enumerate(zip(seq.output, seq.logprobs)):
        row = logits[len(prompt) + t - 1].astype(np.float64)
        p = np.exp(row - row.max())
        p /= p.sum()
        assert info.chosen_id == tok == int(np.argmax(row))
        assert abs(info.chosen_prob - p[tok]) < 1e-4 and abs(info.entropy + (p * np.log(p)).sum()) < 1e-3
        assert [i for i, _ in info.top_candidates] == [int(i) for i in np.argsort(-row, kind="stable")[:4]]
