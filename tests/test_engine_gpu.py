"""The engine against the plain implementation, in 32-bit and in bfloat16,
under every way of cutting the work: each request alone and whole; most of it
in one step and the last 32 tokens one by one; in portions of changing size;
and mixed, up to four live requests with so few pages that they are reused."""
import numpy as np
import pytest
import torch

from helpers import (TINY, TOL, first_wrong, make_folder, plain_logits, random_ids, rel_err, run_trace_on_engine,
                     sharpen_attention, trace_mixed, trace_portions, trace_tail_decoded, trace_whole)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_cache = {}


def _stored(dtype):
    return torch.bfloat16 if dtype == "bfloat16" else torch.float32


def _setup(tmp_path_factory, name, dtype):
    """(folder, model) for a tiny configuration, built once per session.  Configuration C
    (head size 64) gets wider weights and sharpened attention."""
    key = (name, dtype)
    if key not in _cache:
        from gibbs_b200 import load_model
        if name == "C":
            folder = sharpen_attention(make_folder(tmp_path_factory.mktemp("models"), name, stored=_stored(dtype)))
        else:
            folder = make_folder(tmp_path_factory.mktemp("models"), name, stored=_stored(dtype))
        _cache[key] = (folder, load_model(folder, dtype=dtype, device="cuda:0"))
    return _cache[key]


def _requests(name, lengths, seed=0):
    vocab = TINY[name][0]["vocab_size"]
    return {f"r{i}": random_ids(seed * 100 + i, n, vocab) for i, n in enumerate(lengths)}


def _compare(folder, requests, got, dtype):
    worst = 0.0
    for rid, ids in requests.items():
        want = plain_logits(folder, ids)
        assert got[rid].shape == want.shape, rid
        bad = first_wrong(got[rid], want, TOL[dtype])
        assert bad is None, f"request {rid}: first wrong position {bad[0]} of {len(ids)} (rel err {bad[1]:.3g})"
        worst = max(worst, rel_err(got[rid], want))
    return worst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt(tmp_path_factory, name, dtype):
    from gibbs_b200 import Engine
    folder, model = _setup(tmp_path_factory, name, dtype)
    eng = Engine(model, n_pages=32, page_size=16)
    reqs = _requests(name, [1, 7, 40, 150, 300])
    worst = _compare(folder, reqs, run_trace_on_engine(eng, trace_whole(reqs)), dtype)
    print(f"whole {name} {dtype}: worst rel err {worst:.3g}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(tmp_path_factory, name, dtype):
    from gibbs_b200 import Engine
    folder, model = _setup(tmp_path_factory, name, dtype)
    eng = Engine(model, n_pages=16, page_size=16, guard_cache=True)
    assert eng.plan is not None, eng.plan_refusal
    reqs = _requests(name, [33, 100, 177], seed=1)
    worst = _compare(folder, reqs, run_trace_on_engine(eng, trace_tail_decoded(reqs)), dtype)
    print(f"tail {name} {dtype}: worst rel err {worst:.3g}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_changing_size(tmp_path_factory, name, dtype):
    from gibbs_b200 import Engine
    folder, model = _setup(tmp_path_factory, name, dtype)
    eng = Engine(model, n_pages=26, page_size=8, guard_cache=True)
    reqs = _requests(name, [5, 64, 131, 200], seed=2)
    worst = _compare(folder, reqs, run_trace_on_engine(eng, trace_portions(reqs)), dtype)
    print(f"portions {name} {dtype}: worst rel err {worst:.3g}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_page_reuse(tmp_path_factory, name, dtype):
    """Guard pages around every page tensor and guard bytes behind every state slot are checked
    after every step: a write one row past a page or slot is found in the step that made it."""
    from gibbs_b200 import Engine
    folder, model = _setup(tmp_path_factory, name, dtype)
    capacity = 448
    eng = Engine(model, n_pages=capacity // 16, page_size=16, max_requests=4, guard_cache=True)
    assert eng.plan is not None and eng.cache.guard, eng.plan_refusal
    reqs = _requests(name, [90, 37, 128, 61, 150, 2, 75, 100, 33, 119], seed=3)
    steps = trace_mixed(reqs, capacity_tokens=capacity, max_live=4, seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    worst = _compare(folder, reqs, run_trace_on_engine(eng, steps), dtype)
    # every page and slot was handed out more than once
    assert sum(len(v) for v in reqs.values()) > capacity
    print(f"mixed {name} {dtype}: worst rel err {worst:.3g}, {len(steps)} steps")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_random_mixed_traces_without_a_host_wait_between_steps(tmp_path_factory, name, dtype):
    """The traces above look at the device's status after every step, which makes the host wait for
    the step.  Here step follows step as a scheduler launches them (the kernels of a step start while
    the kernel in front still runs, and read what earlier steps left before their dependency is met):
    random requests (lengths at the edges of pages), page sizes and pool sizes, with and without
    decode graphs and the step plan; the logits are collected on the device and compared at the end."""
    from gibbs_b200 import Engine, StepEntry
    folder, model = _setup(tmp_path_factory, name, dtype)
    vocab = TINY[name][0]["vocab_size"]
    for seed in range(1, 13):
        rng = np.random.default_rng(1000 * seed + ord(name))
        lens = [int(rng.choice([1, 2, 15, 16, 17, 31, 33, 63, 64, 65, 100, 129, 200, 257]))
                for _ in range(int(rng.integers(3, 8)))]
        reqs = {f"s{seed}r{i}": random_ids(seed * 100 + i, n, vocab) for i, n in enumerate(lens)}
        page = int(rng.choice([8, 16, 32]))
        cap = max(-(-max(lens) // 64) * 64 + 64, int(rng.choice([192, 320, 448])))
        steps = trace_mixed(reqs, capacity_tokens=cap, max_live=4, seed=seed)
        eng = Engine(model, n_pages=cap // page + 4, page_size=page, max_requests=4,
                     use_graphs=bool(rng.integers(0, 2)), use_plan=bool(rng.integers(0, 4)))
        outs = []
        for s in steps:
            for ent in s["entries"]:
                if not eng.is_live(ent["id"]):
                    eng.open(ent["id"])
            bases = {ent["id"]: eng.length(ent["id"]) for ent in s["entries"]}
            logits = eng.step([StepEntry(ent["id"], ent["tokens"], ent["want"]) for ent in s["entries"]])
            if logits is not None:
                outs.append((s, bases, logits.clone()))      # (a decode graph's logits are overwritten by its next replay)
            for rid in s["end"]:
                eng.close(rid)
        torch.cuda.synchronize()
        eng.check_status()
        eng.cache.check()
        got = {}
        for s, bases, logits in outs:
            arr, row = logits.cpu().numpy(), 0
            for ent in s["entries"]:
                for w in ent["want"]:
                    got.setdefault(ent["id"], {})[bases[ent["id"]] + w] = arr[row]
                    row += 1
        what = f"seed {seed}, pages of {page}, {cap} tokens, graphs {eng.use_graphs}, plan {eng.plan is not None}"
        for rid, ids in reqs.items():
            assert sorted(got[rid]) == list(range(len(ids))), (what, rid)
            bad = first_wrong(np.stack([got[rid][p] for p in range(len(ids))]), plain_logits(folder, ids), TOL[dtype])
            assert bad is None, f"{what}: request {rid} of {len(ids)}: first wrong position {bad[0]} (rel err {bad[1]:.3g})"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_step_plan_gives_the_same_bits_as_the_parts_forward(tmp_path_factory, name, dtype):
    """The same model stepped through the C walker of its plan and through the parts' forward
    methods: one sequence of kernels either way, so the logits are equal bit for bit, under mixed
    batches and decoding (graphs on in both)."""
    from gibbs_b200 import Engine
    folder, model = _setup(tmp_path_factory, name, dtype)
    reqs = _requests(name, [90, 37, 128, 61, 150, 2], seed=7)
    got = []
    for use_plan in (True, False):
        eng = Engine(model, n_pages=28, page_size=16, max_requests=4, use_plan=use_plan)
        assert (eng.plan is not None) == use_plan, eng.plan_refusal
        a = run_trace_on_engine(eng, trace_mixed(reqs, capacity_tokens=448, max_live=4, seed=5))
        b = run_trace_on_engine(eng, trace_tail_decoded({k: v for k, v in list(reqs.items())[:2]}, tail=20))
        got.append((a, b))
        assert not eng.cache.live
    for (pa, pb), (fa, fb) in [(got[0], got[1])]:
        for rid in pa:
            assert np.array_equal(pa[rid], fa[rid]), rid
        for rid in pb:
            assert np.array_equal(pb[rid], fb[rid]), rid


def test_token_ids_are_checked_before_anything_changes(tmp_path_factory):
    """A token id outside the vocabulary, in a short portion or a long one, as a list or as an
    array, is refused with its value; the request stays as it was and the same tokens given as a
    list and as an array give the same logits."""
    from gibbs_b200 import Engine
    from gibbs_b200.engine.step import StepEntry, StepError
    folder, model = _setup(tmp_path_factory, "A", "float32")
    vocab = TINY["A"][0]["vocab_size"]
    eng = Engine(model, n_pages=16, page_size=16, max_requests=2)
    eng.open("a")
    free = eng.cache.free_pages()
    good = random_ids(11, 70, vocab)
    for bad_ids, value in (([3, vocab, 5], vocab), ([-1], -1), (good[:40] + [vocab + 7] + good[40:], vocab + 7),
                           (np.array(good[:50] + [-3], dtype=np.int64), -3)):
        with pytest.raises(StepError, match=f"token id {value} outside the vocabulary"):
            eng.step([StepEntry("a", bad_ids, [0])])
        assert eng.length("a") == 0 and eng.cache.free_pages() == free
    with pytest.raises(StepError, match="integers"):
        eng.step([StepEntry("a", [0.5] * 40, [0])])
    first = eng.step([StepEntry("a", good, [69])]).clone()
    eng.close("a")
    eng.open("b")
    second = eng.step([StepEntry("b", np.array(good, dtype=np.int32), [69])])
    assert torch.equal(first, second)
    eng.close("b")
    eng.cache.check()


@pytest.mark.parametrize("use_graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_tokens_fed_from_the_device_equal_tokens_given_by_the_host(tmp_path_factory, dtype, use_graphs):
    """``Engine.step(..., feed=...)``: ids that lie on the device (where a sampler wrote them) stand
    in for the host's; entries may be fed from any place, beside entries with tokens of their own."""
    from gibbs_b200 import Engine
    from gibbs_b200.engine.step import StepEntry, StepError
    folder, model = _setup(tmp_path_factory, "B", dtype)
    reqs = _requests("B", [20, 9, 33], seed=3)
    picked_host = [17, 999, 4, 321]
    picked = torch.tensor(picked_host, dtype=torch.int32, device="cuda:0")
    out = []
    for fed in (False, True):
        eng = Engine(model, n_pages=24, page_size=16, max_requests=4, use_graphs=use_graphs)
        rows = []
        for rid in reqs:
            eng.open(rid)
        eng.step([StepEntry(rid, toks) for rid, toks in reqs.items()])
        rids = list(reqs)
        for turn in range(3):       # the second and third turn replay the decode graph
            places = [(turn + 2 * i) % 4 for i in range(3)]
            if fed:
                entries = [StepEntry(r, [0], [0]) for r in rids]
                rows.append(eng.step(entries, feed=(picked, places)).clone())
            else:
                rows.append(eng.step([StepEntry(r, [picked_host[p]], [0]) for r, p in zip(rids, places)]).clone())
        # a prompt portion with tokens of its own beside two fed tokens
        portion = random_ids(8, 5, 1000)
        if fed:
            entries = [StepEntry(rids[0], [0], [0]), StepEntry(rids[1], portion, [1, 4]), StepEntry(rids[2], [0], [0])]
            rows.append(eng.step(entries, feed=(picked, [3, -1, 1])).clone())
            with pytest.raises(StepError, match="stands alone"):
                eng.step([StepEntry(rids[0], [1, 2], [0])], feed=(picked, [0]))
            with pytest.raises(StepError, match="stands alone"):
                eng.step([StepEntry(rids[0], [0], [0])], feed=(picked, [4]))
        else:
            entries = [StepEntry(rids[0], [picked_host[3]], [0]), StepEntry(rids[1], portion, [1, 4]),
                       StepEntry(rids[2], [picked_host[1]], [0])]
            rows.append(eng.step(entries).clone())
        eng.check_status()
        out.append(rows)
    for a, b in zip(*out):
        assert torch.equal(a, b)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_cluster_products_with_the_norm_inside_give_the_plain_logits(tmp_path_factory, name, monkeypatch):
    """The other way of running decode-sized products (GIBBS_B200_DECODE_ROWS=16: K split inside a
    thread-block cluster, the norm in front of a product run by the product itself), switched on for
    this test: mixed batches and token-by-token decoding against the plain implementation, and the
    step plan against the parts' forward methods bit for bit."""
    from gibbs_b200 import Engine, ops
    monkeypatch.setattr(ops, "DECODE_ROWS", 16)
    monkeypatch.setattr(ops, "DECODE_PRODUCTS", True)
    folder, model = _setup(tmp_path_factory, name, "bfloat16")
    reqs = _requests(name, [90, 37, 128, 61, 150, 2], seed=11)
    got = []
    for use_plan in (True, False):
        eng = Engine(model, n_pages=28, page_size=16, max_requests=4, use_plan=use_plan, guard_cache=True)
        assert (eng.plan is not None) == use_plan, eng.plan_refusal
        before = ops.launch_count()
        a = run_trace_on_engine(eng, trace_mixed(reqs, capacity_tokens=448, max_live=4, seed=5))
        b = run_trace_on_engine(eng, trace_tail_decoded({k: v for k, v in list(reqs.items())[:2]}, tail=20))
        _compare(folder, reqs, a, "bfloat16")
        _compare(folder, {k: v for k, v in list(reqs.items())[:2]}, b, "bfloat16")
        got.append((a, b))
    for x, y in zip(got[0], got[1]):
        for rid in x:
            assert np.array_equal(x[rid], y[rid]), rid


def test_a_step_packs_only_the_block_table_columns_it_needs(tmp_path_factory):
    """An engine laid out for a very long context (65,536 positions: 4,096 table entries a request)
    copies a few hundred bytes of metadata for a short step, not its tables' full width; only decode
    steps, whose layout a CUDA graph freezes, carry the full width.  The logits are those of an
    engine laid out for a short context."""
    from gibbs_b200 import Engine, StepEntry
    folder, model = _setup(tmp_path_factory, "B", "bfloat16")
    ids = random_ids(3, 60, 1000)
    outs = []
    for ctx in (512, 65536):
        eng = Engine(model, n_pages=16, page_size=16, max_requests=4, max_context=ctx)
        eng.open("a"), eng.open("b")
        rows = [eng.step([StepEntry("a", ids[:37], [36]), StepEntry("b", ids[:5], [4])]).clone()]
        if ctx == 65536:
            offs, total = eng.builder._layout(42, 2, 2, False, 3)
            assert total < 300 and eng.cache.max_blocks == 4096
        for t in ids[37:45]:
            rows.append(eng.step([StepEntry("a", [t], [0]), StepEntry("b", [t], [0])]).clone())
        eng.check_status()
        outs.append(torch.cat(rows))
    assert torch.equal(outs[0], outs[1])
