"""The scheduler's decisions on a fake engine (no GPU).  The invariants follow
the reference's own scheduler tests (MisterTK/gibbs src/scheduler/mod.rs:1632-1931):
decoding never starves, a short prompt is not stuck behind a long one, a long
prompt is not starved, max_new_tokens is exact, generation stops at the
context's end, a cancelled request frees what it holds."""
import pytest

import random

from fake_engine import FakeEngine, LaggingSampler, argmax_sampler, expected_greedy
from gibbs_b200.engine.scheduler import FinishReason, Scheduler
from gibbs_b200.sampling import SamplingParams

GREEDY = SamplingParams(temperature=0.0, max_new_tokens=8)


def _sched(engine, **kw):
    return Scheduler(engine, argmax_sampler, **kw)


def test_generate_matches_the_model_and_frees_everything():
    eng = FakeEngine()
    s = _sched(eng, max_batch_tokens=16)
    prompts = [[3, 4, 5], list(range(1, 41)), [7]]
    outs = s.generate(prompts, GREEDY)
    assert outs == [expected_greedy(p, 8, eng.vocab) for p in prompts]
    assert all(s.sequences[i].finish == FinishReason.LENGTH for i in range(3))
    assert not eng.cache.live and eng.cache.free_pages() == [64] and eng.cache.slots.n_free == 4


def test_token_budget_and_decodes_never_starve():
    eng = FakeEngine(max_context=512)
    s = _sched(eng, max_batch_tokens=10)
    a = s.submit([1, 2], SamplingParams(temperature=0.0, max_new_tokens=30))
    s.step()                                        # a is decoding from now on
    b = s.submit(list(range(1, 101)), GREEDY)
    while s.sequences[b].fed < 100:
        before, left = len(s.sequences[a].output), 100 - s.sequences[b].fed
        s.step()
        step = eng.log[-1]
        assert sum(n for _, n, _ in step) <= 10
        if s.sequences[a].finish is None:
            assert len(s.sequences[a].output) == before + 1      # one token every step
            assert (a, 1, True) in step
            assert dict((r, n) for r, n, _ in step)[b] == min(9, left)   # the rest of the budget goes to the prompt
    s.run()
    assert s.sequences[b].output == expected_greedy(list(range(1, 101)), 8, eng.vocab)


def test_short_prompt_is_not_stuck_behind_a_long_one_and_long_is_not_starved():
    eng = FakeEngine(max_context=512, n_pages=200)
    s = _sched(eng, max_batch_tokens=16)
    long_ = s.submit(list(range(1, 201)), GREEDY)
    s.step()
    short = s.submit([9, 9, 9], GREEDY)
    s.step()
    # the short prompt (shortest remaining first) got its three tokens and its first output
    assert len(s.sequences[short].output) == 1
    # the oldest prefilling request keeps at least half of the budget
    assert dict((r, n) for r, n, _ in eng.log[-1])[long_] >= 8
    for _ in range(40):
        s.submit([5, 6], SamplingParams(temperature=0.0, max_new_tokens=1))
    fed_before = s.sequences[long_].fed
    for _ in range(6):
        s.step()
        assert dict((r, n) for r, n, _ in eng.log[-1]).get(long_, 0) >= 8 or s.sequences[long_].fed >= 200
    assert s.sequences[long_].fed > fed_before
    s.run()
    assert s.sequences[long_].output == expected_greedy(list(range(1, 201)), 8, eng.vocab)


def test_max_new_tokens_is_exact_and_zero_is_allowed():
    eng = FakeEngine()
    s = _sched(eng)
    ids = [s.submit([1, 2, 3], SamplingParams(temperature=0.0, max_new_tokens=n)) for n in (0, 1, 5)]
    s.run()
    assert [len(s.sequences[i].output) for i in ids] == [0, 1, 5]
    assert all(s.sequences[i].finish == FinishReason.LENGTH for i in ids)


def test_stops_at_the_context_end_and_rejects_prompts_that_do_not_fit():
    eng = FakeEngine(max_context=12)
    s = _sched(eng)
    i = s.submit(list(range(1, 9)), SamplingParams(temperature=0.0, max_new_tokens=100))
    assert s.sequences[i].params.max_new_tokens == 4            # clamped at submission
    s.run()
    assert len(s.sequences[i].output) == 4 and s.sequences[i].finish == FinishReason.LENGTH
    with pytest.raises(ValueError, match="context"):
        s.submit(list(range(12)))
    j = s.submit([])                                            # an empty prompt becomes token 1
    assert s.sequences[j].prompt == [1]


def test_stop_ids_are_not_emitted():
    eng = FakeEngine()
    want = expected_greedy([4, 4], 8, eng.vocab)
    eos = want[3]
    cut = want.index(eos)            # the id may occur earlier than the fourth token
    s = _sched(eng, eos_ids=[eos])
    i = s.submit([4, 4], GREEDY)
    s.run()
    assert s.sequences[i].output == want[:cut] and s.sequences[i].finish == FinishReason.STOP
    s2 = _sched(FakeEngine())
    j = s2.submit([4, 4], SamplingParams(temperature=0.0, max_new_tokens=8, stop_ids=(eos,)))
    s2.run()
    assert s2.sequences[j].output == want[:cut]


def test_cancel_frees_pages_and_slot():
    eng = FakeEngine()
    s = _sched(eng, max_batch_tokens=8)
    i = s.submit(list(range(1, 60)), GREEDY)
    k = s.submit([1], GREEDY)
    s.step()
    assert eng.cache.free_pages()[0] < 64
    s.cancel(i)
    w = s.submit([2], GREEDY)
    s.cancel(w)                                                # cancelled while still waiting
    s.run()
    assert s.sequences[i].finish == FinishReason.CANCELLED and s.sequences[w].finish == FinishReason.CANCELLED
    assert s.sequences[k].finish == FinishReason.LENGTH
    assert eng.cache.free_pages() == [64] and eng.cache.slots.n_free == 4 and not eng.cache.live


def test_admission_waits_for_slots_first_come_first_served():
    eng = FakeEngine(max_requests=2)
    s = _sched(eng)
    ids = [s.submit([i + 1], SamplingParams(temperature=0.0, max_new_tokens=3)) for i in range(5)]
    order = []
    while s.has_work():
        out = s.step()
        assert out.active_sequences <= 2 and len(eng.cache.live) <= 2
        order += [i for i, _ in out.finished]
    assert order == ids


def test_pages_run_out_the_last_admitted_is_preempted_and_recomputed():
    # 10 pages of 4 tokens; two requests that each grow to 28 tokens cannot both stay
    eng = FakeEngine(n_pages=10, page_size=4, max_requests=4, max_context=64)
    s = _sched(eng, max_batch_tokens=64)
    p0, p1 = list(range(1, 13)), list(range(20, 32))
    a = s.submit(p0, SamplingParams(temperature=0.0, max_new_tokens=16))
    b = s.submit(p1, SamplingParams(temperature=0.0, max_new_tokens=16))
    emitted, preempted = {a: [], b: []}, []
    while s.has_work():
        out = s.step()
        for i, t in out.emitted:
            emitted[i].append(t)
        preempted += out.preempted
        eng.cache.check()
    assert preempted and set(preempted) == {b}                 # the one admitted last gives way
    assert s.sequences[b].preemptions >= 1
    # tokens are the same as without preemption, and none was emitted twice
    assert emitted[a] == s.sequences[a].output == expected_greedy(p0, 16, eng.vocab)
    assert emitted[b] == s.sequences[b].output == expected_greedy(p1, 16, eng.vocab)
    assert eng.cache.free_pages() == [10] and not eng.cache.live


def test_a_request_that_cannot_fit_alone_ends_with_an_error():
    eng = FakeEngine(n_pages=2, page_size=4, max_context=64)
    s = _sched(eng, max_batch_tokens=64)
    big = s.submit(list(range(1, 20)), GREEDY)                 # first portion needs 5 pages
    grow = s.submit([1, 2, 3], SamplingParams(temperature=0.0, max_new_tokens=30))   # outgrows 2 pages
    s.run(max_steps=200)
    assert s.sequences[big].finish == FinishReason.ERROR and "pool" in s.sequences[big].error
    assert s.sequences[grow].finish == FinishReason.ERROR and len(s.sequences[grow].output) >= 5
    assert eng.cache.free_pages() == [2] and not eng.cache.live


def test_a_failing_step_ends_its_requests_with_an_error_and_the_loop_goes_on():
    eng = FakeEngine(fail_on=1)
    s = _sched(eng)
    a = s.submit([1, 2, 3], GREEDY)
    s.step()
    out = s.step()
    assert (a, FinishReason.ERROR) in out.finished and "injected" in s.sequences[a].error
    assert not eng.cache.live
    b = s.submit([1, 2, 3], GREEDY)
    s.run()
    assert s.sequences[b].output == expected_greedy([1, 2, 3], 8, eng.vocab)


def test_seeds_are_per_request_and_reproducible():
    s1, s2 = _sched(FakeEngine(), seed=5), _sched(FakeEngine(), seed=5)
    ids1 = [s1.submit([1]), s1.submit([1], SamplingParams(seed=99))]
    ids2 = [s2.submit([1]), s2.submit([1], SamplingParams(seed=99))]
    assert [s1.sequences[i].seed for i in ids1] == [s2.sequences[i].seed for i in ids2]
    assert s1.sequences[ids1[0]].seed != s1.sequences[ids1[1]].seed == 99


# ---------------------------------------------------------------- token feedback (overlap)
def _lagging(engine, **kw):
    return Scheduler(engine, LaggingSampler(engine), overlap=True, **kw)


def test_overlap_launches_the_next_decode_step_before_it_reads_the_last():
    eng = FakeEngine()
    s = _lagging(eng, max_batch_tokens=16)
    prompts = [[3, 4, 5], list(range(1, 31)), [7]]
    outs = s.generate(prompts, GREEDY)
    assert outs == [expected_greedy(p, 8, eng.vocab) for p in prompts]
    ev = eng.events
    fed = [i for i, e in enumerate(ev) if e == "launch fed"]
    assert len(fed) >= 6
    # every fed launch went out while the ids of the step before were still unread
    for i in fed:
        assert ev[:i].count("read") == sum(1 for e in ev[:i] if e.startswith("launch")) - 1
    assert not eng.cache.live and eng.cache.free_pages() == [64] and eng.cache.slots.n_free == 4


def test_overlap_drops_the_token_after_an_unforeseen_end_and_foresees_ends_by_length():
    eng = FakeEngine()
    want = expected_greedy([4, 4], 12, eng.vocab)
    eos = want[5]
    cut = want.index(eos)
    s = _lagging(eng, eos_ids=[eos])
    i = s.submit([4, 4], SamplingParams(temperature=0.0, max_new_tokens=12))
    j = s.submit([9, 1, 1], SamplingParams(temperature=0.0, max_new_tokens=3))
    emitted = {i: [], j: []}
    while s.has_work():
        for k, t in s.step().emitted:
            emitted[k].append(t)
    assert emitted[i] == s.sequences[i].output == want[:cut] and s.sequences[i].finish == FinishReason.STOP
    want_j = expected_greedy([9, 1, 1], 3, eng.vocab, eos=[eos])
    assert emitted[j] == s.sequences[j].output == want_j
    # the request that ends by length was fed exactly its prompt and its tokens but the last
    assert eng.events.count("launch fed") >= 2
    assert not eng.cache.live and eng.cache.free_pages() == [64] and eng.cache.slots.n_free == 4


def test_overlap_gives_way_to_admission_cancellation_and_preemption():
    # the preemption scenario of the test above, with ids that lag
    eng = FakeEngine(n_pages=10, page_size=4, max_requests=4, max_context=64)
    s = _lagging(eng, max_batch_tokens=64)
    p0, p1 = list(range(1, 13)), list(range(20, 32))
    a = s.submit(p0, SamplingParams(temperature=0.0, max_new_tokens=16))
    b = s.submit(p1, SamplingParams(temperature=0.0, max_new_tokens=16))
    emitted, preempted = {a: [], b: []}, []
    while s.has_work():
        out = s.step()
        for i, t in out.emitted:
            emitted[i].append(t)
        preempted += out.preempted
        eng.cache.check()
    assert set(preempted) == {b}
    assert emitted[a] == expected_greedy(p0, 16, eng.vocab) and emitted[b] == expected_greedy(p1, 16, eng.vocab)
    assert eng.cache.free_pages() == [10] and not eng.cache.live
    # a request that arrives while a step is in flight is admitted at the next step
    eng = FakeEngine()
    s = _lagging(eng)
    a = s.submit([1, 2, 3], SamplingParams(temperature=0.0, max_new_tokens=20))
    for _ in range(4):
        s.step()
    b = s.submit([5, 6], GREEDY)
    s.step()
    s.step()
    assert eng.is_open(b) if hasattr(eng, "is_open") else b in eng.cache.live
    s.cancel(a)
    s.run()
    assert s.sequences[a].finish == FinishReason.CANCELLED
    assert s.sequences[a].output == expected_greedy([1, 2, 3], 20, eng.vocab)[:len(s.sequences[a].output)]
    assert s.sequences[b].output == expected_greedy([5, 6], 8, eng.vocab)
    assert not eng.cache.live and eng.cache.free_pages() == [64]


@pytest.mark.parametrize("seed", range(6))
def test_overlap_emits_what_the_plain_loop_emits_under_random_traffic(seed):
    def run(overlap):
        rng = random.Random(seed)
        eng = FakeEngine(n_pages=rng.choice([14, 24, 64]), page_size=4, max_requests=3, max_context=48, vocab=11)
        sampler = LaggingSampler(eng)
        s = Scheduler(eng, sampler, max_batch_tokens=rng.choice([6, 16]), eos_ids=[3], overlap=overlap)
        ids, emitted = [], {}
        for step in range(400):
            if step < 60 and rng.random() < 0.3:
                prompt = [rng.randrange(11) for _ in range(rng.randint(1, 14))]
                ids.append(s.submit(prompt, SamplingParams(temperature=0.0, max_new_tokens=rng.randint(0, 12))))
            if not s.has_work():
                if step >= 60:
                    break
                continue
            for i, t in s.step().emitted:
                emitted.setdefault(i, []).append(t)
            eng.cache.check()
        assert not s.has_work() and not eng.cache.live
        assert all(emitted.get(i, []) == s.sequences[i].output for i in ids)
        return [(s.sequences[i].output, s.sequences[i].finish) for i in ids], eng.events.count("launch fed")

    plain, none_fed = run(False)
    lagging, fed = run(True)
    assert none_fed == 0 and fed > 0
    assert plain == lagging


@pytest.mark.parametrize("fail_on", [1, 2, 3, 5])
def test_a_failing_fed_step_ends_its_requests_like_a_failing_plain_step(fail_on):
    """The same engine step fails with and without token feedback: the same requests end with
    ``error`` after the same tokens, nothing stays reserved, and the loop goes on."""
    def run(overlap):
        eng = FakeEngine(fail_on=fail_on, n_pages=16, page_size=4)
        s = Scheduler(eng, LaggingSampler(eng), overlap=overlap)
        a = s.submit([1, 2, 3], SamplingParams(temperature=0.0, max_new_tokens=12))
        b = s.submit([5, 6, 7, 8, 9], SamplingParams(temperature=0.0, max_new_tokens=12))
        emitted = {a: [], b: []}
        while s.has_work():
            for i, t in s.step().emitted:
                emitted[i].append(t)
            eng.cache.check()
        assert not eng.cache.live and eng.cache.free_pages() == [16] and eng.cache.slots.n_free == 4
        assert emitted == {i: s.sequences[i].output for i in (a, b)}
        for i in (a, b):
            assert s.sequences[i].finish == FinishReason.ERROR and "injected" in s.sequences[i].error
        # the loop goes on with a new request
        c = s.submit([4, 4], GREEDY)
        s.run()
        assert s.sequences[c].output == expected_greedy([4, 4], 8, eng.vocab)
        return [(s.sequences[i].output, s.sequences[i].finish) for i in (a, b)], eng.events.count("launch fed")

    plain, none_fed = run(False)
    lagging, fed = run(True)
    assert none_fed == 0 and (fed > 0 or fail_on < 2)
    assert plain == lagging


def test_a_sampler_that_fails_after_a_fed_step_ends_the_requests():
    """The engine has advanced when the sampler raises: the requests cannot be stepped again at
    the old position, so they end with ``error`` and give everything back."""
    eng = FakeEngine()

    class Flaky(LaggingSampler):
        calls = 0

        def sample_async(self, *a):
            Flaky.calls += 1
            if Flaky.calls == 3:
                raise RuntimeError("sampler fell over")
            return super().sample_async(*a)

    s = Scheduler(eng, Flaky(eng), overlap=True)
    a = s.submit([1, 2, 3], SamplingParams(temperature=0.0, max_new_tokens=12))
    s.run()
    assert s.sequences[a].finish == FinishReason.ERROR and "fell over" in s.sequences[a].error
    assert s.sequences[a].output == expected_greedy([1, 2, 3], 12, eng.vocab)[:len(s.sequences[a].output)]
    assert len(s.sequences[a].output) >= 2
    assert not eng.cache.live and eng.cache.free_pages() == [64]


# ---------------------------------------------------------------- measured prompt budget
def test_prefill_tuner_rules():
    """The budget rules of the reference's PrefillTuner (src/scheduler/mod.rs:350-403)."""
    from gibbs_b200.engine.scheduler import PrefillTuner
    t = PrefillTuner()
    assert t.budget(False) == 64 and t.budget(True) == 64          # nothing timed yet
    t.record((0.010, 100), (0.0, 0))                               # 100 us a prompt token
    assert t.budget(True) == 1                                     # no decode round timed: the step is the decoders'
    assert t.budget(False) == 1000                                 # about 100 ms of prompt when nothing decodes
    t.record((0.0, 0), (0.002, 4))                                 # a decode round of 2 ms
    assert t.budget(True) == 20                                    # as many prompt tokens as cost one decode round
    t.record((0.030, 100), (0.0, 0))                               # 300 us a token: 0.75 * 100 + 0.25 * 300 = 150
    assert abs(t.prefill_s_per_token - 150e-6) < 1e-12 and t.budget(True) == 13
    t.record((0.5, 10), (0.5, 3))                                  # a mixed step tells neither cost: not recorded
    assert abs(t.prefill_s_per_token - 150e-6) < 1e-12 and t.decode_round_s == 0.002
    fast = PrefillTuner()
    fast.record((1e-6, 100), (0.0, 0))
    assert fast.budget(False) == 2048                              # clamped to the largest portion
    slow = PrefillTuner()
    slow.record((10.0, 1), (0.0, 0))
    slow.record((0.0, 0), (0.001, 1))
    assert slow.budget(True) == 1                                  # never below one token
    assert PrefillTuner(whole_prompt=True).budget(True) > 1 << 20


def test_scheduler_sizes_prompt_portions_from_measured_costs():
    """With a tuner, the scheduler times its steps and cuts prompt portions to cost about one decode
    round while requests decode; the clock here is the fake engine's: 50 us a prompt token, 1 ms a
    decode round."""
    from gibbs_b200.engine.scheduler import PrefillTuner

    class Clocked(FakeEngine):
        now = 0.0

        def step(self, entries, feed=None):
            n_prompt = sum(len(e.tokens) for e in entries if len(e.tokens) > 1)
            self.now += 50e-6 * n_prompt + (1e-3 if any(len(e.tokens) == 1 for e in entries) else 0.0)
            return super().step(entries, feed)

    eng = Clocked(n_pages=400, page_size=4, max_requests=4, max_context=1024)
    tuner = PrefillTuner()
    s = Scheduler(eng, argmax_sampler, max_batch_tokens=512, tuner=tuner, clock=lambda: eng.now)
    a = s.submit([7, 8, 9], SamplingParams(temperature=0.0, max_new_tokens=40))
    s.step()                                        # 3 prompt tokens: the first prefill is timed
    assert abs(tuner.prefill_s_per_token - 50e-6) < 1e-9
    s.step()                                        # a pure decode round is timed
    assert abs(tuner.decode_round_s - 1e-3) < 1e-9
    b = s.submit(list(range(1, 301)), GREEDY)
    portions = []
    while s.sequences[b].fed < 300:
        before = s.sequences[b].fed
        s.step()
        portions.append(s.sequences[b].fed - before)
    # one decode round (1 ms) buys 20 prompt tokens at 50 us each: every portion is that, the last the rest
    assert portions[:-1] == [20] * (len(portions) - 1) and 0 < portions[-1] <= 20 and sum(portions) == 300
    s.run()
    assert s.sequences[a].output == expected_greedy([7, 8, 9], 40, eng.vocab)
    assert s.sequences[b].output == expected_greedy(list(range(1, 301)), 8, eng.vocab)
    # nothing decoding: about 100 ms of prompt (2,000 tokens), capped by the engine's own limit of 512
    c = s.submit(list(range(1, 801)), GREEDY)
    s.step()
    assert s.sequences[c].fed == 512


def test_top_logprobs_are_reported_for_the_requests_that_ask():
    """A request with ``top_logprobs`` gets, per emitted token, its probability, that many
    candidates and the entropy (src/scheduler/mod.rs:272-315, 414-423); its neighbour in the batch
    gets none; with token feedback on, a step with such a request is read at once."""
    from fake_engine import fake_logprob_info
    eng = FakeEngine()
    sampler = LaggingSampler(eng)
    sampler.logprob_info = fake_logprob_info
    s = Scheduler(eng, sampler, overlap=True)
    a = s.submit([3, 4, 5], SamplingParams(temperature=0.0, max_new_tokens=6, top_logprobs=3))
    b = s.submit([9, 9], SamplingParams(temperature=0.0, max_new_tokens=6))
    reported = []
    while s.has_work():
        reported += s.step().logprobs
    assert s.sequences[a].output == expected_greedy([3, 4, 5], 6, eng.vocab)
    assert s.sequences[b].output == expected_greedy([9, 9], 6, eng.vocab)
    infos = s.sequences[a].logprobs
    assert [sid for sid, _ in reported] == [a] * 6 and [i for _, i in reported] == infos and not s.sequences[b].logprobs
    for tok, info in zip(s.sequences[a].output, infos):
        assert info.chosen_id == tok and len(info.top_candidates) == 3 and info.top_candidates[0][0] == tok
        assert 0 < info.chosen_prob < 1 and info.entropy > 0
        assert abs(info.top_candidates[0][1] - info.chosen_prob) < 1e-9
    assert "launch fed" not in eng.events            # every step held a request whose logits had to be read
    with pytest.raises(ValueError, match="top_logprobs"):
        SamplingParams(top_logprobs=0)


def test_sampling_params_top_k_zero_means_off_and_bounds_are_checked():
    """top_k 0 switches the narrower limit off: the sampler then keeps all the candidates it can
    hold (64) and top_p alone cuts them; anything outside 0..64 is refused."""
    assert SamplingParams(top_k=0).resolved_top_k == 64
    assert SamplingParams(top_k=1).resolved_top_k == 1
    assert SamplingParams().resolved_top_k == 50
    for bad in (-1, 65):
        with pytest.raises(ValueError):
            SamplingParams(top_k=bad)


def test_repetition_penalty_gets_the_latest_64_tokens_and_is_not_lagged():
    """A request with a repetition penalty hands the sampler the last 64 tokens of prompt +
    generated text with every pick (MisterTK/gibbs src/scheduler/mod.rs:34-36, 79) and is sampled
    with every id known on the host (no fed step); its neighbour without a penalty passes nothing."""
    eng = FakeEngine(max_context=512, n_pages=200)
    seen = []

    class Recorder(LaggingSampler):
        def __call__(self, logits, params, seeds, counters, recent=None):
            seen.append((list(params), None if recent is None else [list(r) for r in recent]))
            return argmax_sampler(logits, params, seeds, counters)

    s = Scheduler(eng, Recorder(eng), max_batch_tokens=256, overlap=True)
    prompt = list(range(1, 81))
    pen = s.submit(prompt, SamplingParams(temperature=0.0, max_new_tokens=5, repetition_penalty=1.3))
    off = s.submit([4, 5, 6], SamplingParams(temperature=0.0, max_new_tokens=5))
    s.run()
    out = s.sequences[pen].output
    assert len(out) == 5 and len(s.sequences[off].output) == 5
    picks = [(p, r) for p, r in seen if any(q.penalizes for q in p)]
    assert len(picks) == 5                                    # every token of the penalised request came this way
    for n, (params, recent) in enumerate(picks):
        rows = [r for q, r in zip(params, recent) if q.penalizes]
        assert rows == [(prompt + out[:n])[-64:]]
        assert all(r == [] for q, r in zip(params, recent) if not q.penalizes)
    assert eng.cache.check() is None and not eng.cache.live
