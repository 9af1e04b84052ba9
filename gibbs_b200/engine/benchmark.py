"""Measurement of prefill and decode throughput, shared by ``bench.py`` and the
command line's ``--bench``.

Method after MisterTK/gibbs ``src/bench.rs:219-322``: warm-up, then timed
decode steps; the roofline of a decode step is the bytes it must read (every
weight once, and the cache of the live requests) over the memory bandwidth
(``src/bench.rs:298-308``, ``src/graph/program.rs:330-341``).  Times are taken
with CUDA events on the launching stream, after a synchronise.
"""
from __future__ import annotations

import json
import statistics
import subprocess
import threading
import time
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..sampling import Sampler, SamplingParams
from .scheduler import Scheduler
from .step import Engine, StepEntry

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks(path=None) -> dict:
    """Copy bandwidth (GB/s) and bf16 matrix throughput (TFLOP/s) to relate
    measurements to: from the JSON file ``path`` (keys ``hbm_gbs``,
    ``bf16_tflops``, optionally ``bf16_tflops_sustained``; a folder stands for
    its ``MEASURED_PEAKS.json``) when it exists, else the stated fallback
    figures."""
    p = Path(path) if path is not None else None
    if p is not None and p.is_dir():
        p = p / "MEASURED_PEAKS.json"
    if p is not None and p.exists():
        try:
            d = json.loads(p.read_text())
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed
    region runs (reading only; nothing is set)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0, period_ms: int = 20):
        self.index, self.period_ms = index, period_ms
        self.proc, self.lines = None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._read, daemon=True)
            self._t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def model_flops_per_token(model) -> int:
    """Multiply-adds x2 of every projection a token passes through (the head
    is counted separately, per wanted row)."""
    head = model.head.proj.weight
    total = 0
    seen = {head.data_ptr()}
    for b in model.blocks:
        for holder in b.parts.values():
            for v in vars(holder).values():
                w = getattr(v, "weight", None)
                if isinstance(w, torch.Tensor) and w.dim() == 2 and w.data_ptr() not in seen:
                    seen.add(w.data_ptr())
                    total += 2 * w.numel()
    return total


def prefill_flops(model, n_tokens: int, n_logit_rows: int = 1) -> int:
    fl = model_flops_per_token(model) * n_tokens + 2 * model.head.proj.weight.numel() * n_logit_rows
    for b in model.blocks:
        for m in b.parts.values():
            # a part that attends says how many flops its scores and weighted values cost
            extra = getattr(m, "attention_flops", None)
            if extra is not None:
                fl += int(extra(n_tokens))
    return fl


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def measure_prefill(engine: Engine, n_tokens: int, warmup: int = 3, runs: int = 5, seed: int = 0) -> dict:
    """Time from the first token of a whole prompt to its last-row logits, one step."""
    rng = np.random.default_rng(seed)
    times = []
    for i in range(warmup + runs):
        ids = rng.integers(0, engine.vocab_size, n_tokens).tolist()
        engine.open("prefill-bench")
        torch.cuda.synchronize()
        a, b = _events()
        a.record()
        engine.step([StepEntry("prefill-bench", ids, [n_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        engine.close("prefill-bench")
        if i >= warmup:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    return {"ms": ms, "tokens": n_tokens, "value": n_tokens / (ms / 1e3)}


def fill_contexts(engine: Engine, batch: int, prompt_len: int, seed: int, chunk: int = 2048) -> list:
    """Open ``batch`` requests and run their random prompts; returns the ids
    picked greedily from the last prompt position of each."""
    rng = np.random.default_rng(seed)
    sampler = Sampler(engine.device)
    first = []
    for r in range(batch):
        ids = rng.integers(0, engine.vocab_size, prompt_len).tolist()
        engine.open(("bench", r))
        for lo in range(0, prompt_len, chunk):
            part = ids[lo:lo + chunk]
            last = lo + chunk >= prompt_len
            logits = engine.step([StepEntry(("bench", r), part, [len(part) - 1] if last else [])])
        first.append(sampler(logits, [SamplingParams(temperature=0.0)], [0], [0])[0])
    return first


def measure_decode(engine: Engine, batch: int, prompt_len: int, steps: int, warmup: int, seed: int = 0,
                   repeats: int = 1) -> dict:
    """``steps`` decode steps of ``batch`` requests whose contexts start at
    ``prompt_len``: every step feeds each request the token the step before
    picked for it (the ids stay on the device, as in the scheduler's
    overlapped loop), takes the logits and picks the next token greedily on
    the device.  The host copies each step's metadata and launches; it waits
    for nothing inside the timed region.  The region of ``steps`` steps is
    timed ``repeats`` times back to back; the figures are those of the median
    region, ``spread`` is (slowest - fastest) / median."""
    first = fill_contexts(engine, batch, prompt_len, seed)
    sampler = Sampler(engine.device)
    greedy = [SamplingParams(temperature=0.0)] * batch
    zeros = [0] * batch
    places = list(range(batch))
    entries = [StepEntry(("bench", r), [0], [0]) for r in range(batch)]
    tokens = torch.tensor(first, dtype=torch.int32, device=engine.device)

    def one_step(tokens):
        logits = engine.step(entries, feed=(tokens, places))
        return sampler.sample_device(logits, greedy, zeros, zeros)

    for _ in range(warmup):
        tokens = one_step(tokens)
    regions = []
    for _ in range(max(1, repeats)):
        launches0 = ops.launch_count()
        torch.cuda.synchronize()
        a, b = _events()
        t0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            tokens = one_step(tokens)
        b.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        ctx = [engine.length(("bench", r)) - steps // 2 for r in range(batch)]      # mid-region contexts
        regions.append((a.elapsed_time(b), wall, ctx, ops.launch_count() - launches0))
    regions.sort(key=lambda r: r[0])
    ms, wall, ctx, launches = regions[len(regions) // 2]
    spread = (regions[-1][0] - regions[0][0]) / ms
    bytes_step = engine.model.weight_bytes_per_step(batch) + sum(ctx) * engine.cache.kv_bytes_per_token() \
        + batch * engine.cache.slot_bytes
    for r in range(batch):
        engine.close(("bench", r))
    return {"batch": batch, "steps": steps, "ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3),
            "wall_ms_per_step": wall * 1e3 / steps, "bytes_per_step": bytes_step,
            "gbs": bytes_step / (ms / steps / 1e3) / 1e9, "launches": launches,
            "context": int(statistics.mean(ctx)), "repeats": len(regions), "spread": spread}


def decode_kind_shares(engine: Engine, batch: int, prompt_len: int, steps: int = 8, seed: int = 0) -> dict:
    """Which kinds of operation a decode step's time goes to: ``steps`` decode steps of ``batch``
    requests run in the engine's timing mode (every operation bracketed by CUDA events, no CUDA
    graph, operations one after the other), and each kind's share of the summed time is returned
    ({"linear:gate_up": 0.31, "rmsnorm": 0.12, ...}; the reference's per-kernel-class table,
    MisterTK/gibbs src/graph/metal.rs:143-148).  Empty when the model has no step plan."""
    if engine.plan is None:
        return {}
    first = fill_contexts(engine, batch, prompt_len, seed)
    entries = [StepEntry(("bench", r), [t], [0]) for r, t in enumerate(first)]
    graphs, timing = engine.use_graphs, engine.timing
    engine.use_graphs, engine.timing = False, True
    engine.plan.set_timing(True)
    try:
        for _ in range(steps):
            engine.step(entries)
        table = engine.plan.timing_table()
    finally:
        engine.plan.set_timing(False)
        engine.use_graphs, engine.timing = graphs, timing
        for r in range(batch):
            engine.close(("bench", r))
    total = sum(ms for _, ms in table.values()) or 1.0
    return {k: round(ms / total, 4) for k, (_, ms) in sorted(table.items(), key=lambda kv: -kv[1][1])}


def measure_decode_e2e(generator, batch: int, prompt_len: int, steps: int, warmup: int, seed: int = 0,
                       repeats: int = 1) -> dict:
    """The same through the public entry point's scheduler: prompts come from host
    lists, every step copies its metadata (positions, block tables, places of the fed
    ids) from pinned host memory and the picked ids go back to pinned host memory, from
    where they are emitted; a decode step is launched on the ids the device picked one
    step before the host reads them.  ``repeats`` regions of ``steps`` steps are timed back
    to back; the figures are the median region's, ``spread`` is (slowest - fastest) / median."""
    rng = np.random.default_rng(seed)
    sched: Scheduler = generator.scheduler(stop_at_eos=False)
    repeats = max(1, repeats)
    # prompts finish at different steps: leave room so that nobody reaches max_new_tokens while timed
    params = SamplingParams(temperature=0.0, max_new_tokens=warmup + repeats * steps + 4 * batch + 16)
    for _ in range(batch):
        sched.submit(rng.integers(0, generator.engine.vocab_size, prompt_len).tolist(), params)
    while any(not s.output for s in sched.sequences.values()):
        sched.step()
    for _ in range(warmup):
        sched.step()
    regions = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n = 0
        for _ in range(steps):
            n += sched.step().tokens_generated
        torch.cuda.synchronize()
        regions.append((time.perf_counter() - t0, n))
    regions.sort(key=lambda r: r[0] / max(r[1], 1))
    dt, n = regions[len(regions) // 2]
    spread = (regions[-1][0] - regions[0][0]) / dt
    for sid in list(sched.sequences):
        sched.cancel(sid)
    sched.step()
    meta_ints = 4 * 4 * ((batch + 3) // 4) + 6 * 4 * ((batch + 3) // 4) \
        + len(generator.engine.cache.groups) * batch * generator.engine.cache.max_blocks
    return {"value": n / dt, "unit": "tokens/s", "h2d_bytes_per_step": 4 * meta_ints, "d2h_bytes_per_step": 4 * batch,
            "ms_per_step": dt * 1e3 / steps, "repeats": repeats, "spread": spread}


def measure_serving(generator, n_requests: int, min_len: int, max_len: int, new_tokens: int, temperature: float,
                    seed: int = 0) -> dict:
    """Continuous batching end to end: ``n_requests`` prompts of uniform-random length arrive at
    once, are prefilled in portions under the scheduler's token budget while earlier ones decode,
    and each generates ``new_tokens`` tokens by temperature sampling."""
    rng = np.random.default_rng(seed)
    sched: Scheduler = generator.scheduler(stop_at_eos=False)
    lens = rng.integers(min_len, max_len + 1, n_requests)
    params = SamplingParams(temperature=temperature, max_new_tokens=new_tokens, seed=seed)
    for n in lens:
        sched.submit(rng.integers(0, generator.engine.vocab_size, int(n)).tolist(), params)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = prefill_tokens = decoded = preempted = 0
    while sched.has_work():
        out = sched.step()
        steps += 1
        prefill_tokens += out.prefill[1]
        decoded += out.tokens_generated
        preempted += len(out.preempted)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    done = [s for s in sched.sequences.values() if s.finish is not None and s.finish.value == "length"]
    return {"requests": n_requests, "finished_length": len(done), "prompt_tokens": int(lens.sum()),
            "generated_tokens": decoded, "seconds": dt, "steps": steps, "preemptions": preempted,
            "generated_tok_s": decoded / dt, "total_tok_s": (int(lens.sum()) + decoded) / dt}
