"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read
back from <out>/<step>.f32."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, first_wrong, make_folder, plain_logits, random_ids, trace_mixed, trace_tail_decoded

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run(folder, dtype, steps, out, max_tokens, env=None):
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(max_tokens)],
        input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600,
        env=None if env is None else {**os.environ, **env})
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return proc


def _collect(steps, out, vocab):
    got, pos = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        f = Path(out) / f"{s['step']}.f32"
        if n_want == 0:
            assert not f.exists()
            for e in s["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
            continue
        arr = np.fromfile(f, dtype="<f4").reshape(n_want, vocab)
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = arr[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    return got


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("bfloat16", "B")])
def test_trace_run_mixed_and_sparse_wants(tmp_path, dtype, name):
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, name, stored=stored)
    vocab = TINY[name][0]["vocab_size"]
    reqs = {f"q{i}": random_ids(40 + i, n, vocab) for i, n in enumerate([70, 45, 130, 64, 20, 99])}
    steps = trace_mixed(reqs, capacity_tokens=384, max_live=4, seed=9)
    # ask for only some places: every third wanted place is dropped, some steps want nothing
    for k, s in enumerate(steps):
        for e in s["entries"]:
            e["want"] = [] if k % 5 == 4 else [w for w in e["want"] if (w + k) % 3]
    out = tmp_path / "out"
    _run(folder, dtype, steps, out, max_tokens=384)
    got = _collect(steps, out, vocab)
    for rid, ids in reqs.items():
        want = plain_logits(folder, ids)
        rows = sorted(got[rid])
        bad = first_wrong(np.stack([got[rid][p] for p in rows]), want[rows], TOL[dtype])
        assert bad is None, f"{rid}: first wrong wanted place {rows[bad[0]]} (rel err {bad[1]:.3g})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_without_programmatic_dependent_launch(tmp_path, dtype):
    """The kernels read what they can before their dependency wait (metadata, weights, cache and state
    of earlier steps) so that a step's kernels overlap; with GIBBS_B200_PDL=0 every kernel starts
    after the one in front has ended.  Both ways must give the plain implementation's logits: a
    difference between them would be a read that was moved in front of the wait by mistake."""
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, "C", stored=stored)
    vocab = TINY["C"][0]["vocab_size"]
    reqs = {f"q{i}": random_ids(60 + i, n, vocab) for i, n in enumerate([90, 33, 150, 64])}
    steps = trace_mixed(reqs, capacity_tokens=320, max_live=4, seed=4)
    want = {rid: plain_logits(folder, ids) for rid, ids in reqs.items()}
    results = {}
    for mode, env in (("serial", {"GIBBS_B200_PDL": "0"}), ("overlapped", {"GIBBS_B200_PDL": "1"})):
        out = tmp_path / f"out_{mode}"
        _run(folder, dtype, steps, out, max_tokens=320, env=env)
        got = results[mode] = _collect(steps, out, vocab)
        for rid in reqs:
            rows = sorted(got[rid])
            bad = first_wrong(np.stack([got[rid][p] for p in rows]), want[rid][rows], TOL[dtype])
            assert bad is None, f"{mode}, {rid}: first wrong place {rows[bad[0]]} (rel err {bad[1]:.3g})"
    # the same kernels add in the same order either way: the two runs agree to the bit
    for rid in reqs:
        for p in sorted(results["serial"][rid]):
            assert np.array_equal(results["serial"][rid][p], results["overlapped"][rid][p]), (rid, p)


def test_trace_run_fresh_env(tmp_path):
    """Runs with an empty HOME and no inherited python path."""
    folder = make_folder(tmp_path, "A")
    vocab = TINY["A"][0]["vocab_size"]
    reqs = {"only": random_ids(7, 50, vocab)}
    steps = trace_tail_decoded(reqs, tail=8)
    home = tmp_path / "home"
    home.mkdir()
    env = {k: v for k, v in os.environ.items() if k not in ("PYTHONPATH",)}
    env["HOME"] = str(home)
    proc = subprocess.run(
        [str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o"),
         "--max-tokens", "64"],
        input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600, env=env,
        cwd=str(tmp_path))
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = _collect(steps, tmp_path / "o", vocab)
    want = plain_logits(folder, reqs["only"])
    assert first_wrong(np.stack([got["only"][p] for p in sorted(got["only"])]), want, TOL["float32"]) is None
