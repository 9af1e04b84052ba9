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


def _decode_stepper(engine: Engine, batch: int, prompt_len: int, seed: int):
    """Requests with ``prompt_len``-token contexts and a function that runs one fed decode step."""
    first = fill_contexts(engine, batch, prompt_len, seed)
    sampler = Sampler(engine.device)
    greedy, zeros, places = [SamplingParams(temperature=0.0)] * batch, [0] * batch, list(range(batch))
    entries = [StepEntry(("bench", r), [0], [0]) for r in range(batch)]
    state = {"tokens": torch.tensor(first, dtype=torch.int32, device=engine.device)}

    def one_step():
        logits = engine.step(entries, feed=(state["tokens"], places))
        state["tokens"] = sampler.sample_device(logits, greedy, zeros, zeros)

    def close():
        for r in range(batch):
            engine.close(("bench", r))

    return one_step, close


def decode_timeline(engine: Engine, batch: int, prompt_len: int, seed: int = 0) -> list:
    """Start and duration of every kernel of ONE decode step as it runs inside the replayed CUDA
    graph, overlapping as programmatic dependent launch lets them (kernel records from CUPTI,
    through torch.profiler).  Returns rows (name, grid, start_us, dur_us, adds_us): ``adds`` is how
    far the kernel's end lies behind the latest end before it, i.e. what it adds to the chain of
    dependent launches.  A measurement aid: the profiler slows the step down a little, so the
    shares are what to read, not the sum."""
    from torch.profiler import ProfilerActivity, profile
    import tempfile
    one_step, close = _decode_stepper(engine, batch, prompt_len, seed)
    for _ in range(6):
        one_step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(4):
            one_step()
        torch.cuda.synchronize()
    close()
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "trace.json"
        prof.export_chrome_trace(str(path))
        events = [e for e in json.loads(path.read_text())["traceEvents"] if e.get("cat") == "kernel"]
    events.sort(key=lambda e: e["ts"])
    marks = [i for i, e in enumerate(events) if "feed_tokens" in e["name"]]       # the first kernel of a fed step
    step = events[marks[2]:marks[3]]
    t0 = prev_end = step[0]["ts"]
    rows = []
    for e in step:
        end = e["ts"] + e["dur"]
        rows.append((e["name"], tuple(e["args"].get("grid", ())), e["ts"] - t0, e["dur"], end - prev_end))
        prev_end = max(prev_end, end)
    return rows


def prefill_timeline(engine: Engine, n_tokens: int, seed: int = 0) -> list:
    """The same for ONE prompt step of ``n_tokens`` tokens (launched kernel by kernel, not from a
    graph): rows (name, grid, start_us, dur_us, adds_us)."""
    from torch.profiler import ProfilerActivity, profile
    import tempfile
    rng = np.random.default_rng(seed)

    def one_step():
        ids = rng.integers(0, engine.vocab_size, n_tokens).tolist()
        engine.open("prefill-timeline")
        engine.step([StepEntry("prefill-timeline", ids, [n_tokens - 1])])
        torch.cuda.synchronize()
        engine.close("prefill-timeline")

    for _ in range(3):
        one_step()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        one_step()
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "trace.json"
        prof.export_chrome_trace(str(path))
        events = [e for e in json.loads(path.read_text())["traceEvents"] if e.get("cat") == "kernel"]
    events.sort(key=lambda e: e["ts"])
    first = next(i for i, e in enumerate(events) if "embed_kernel" in e["name"])
    step = events[first:]
    t0 = prev_end = step[0]["ts"]
    rows = []
    for e in step:
        end = e["ts"] + e["dur"]
        rows.append((e["name"], tuple(e["args"].get("grid", ())), e["ts"] - t0, e["dur"], end - prev_end))
        prev_end = max(prev_end, end)
    return rows


def prompt_product_times(cfg, n_tokens: int, peak_tflops: float, device="cuda:0") -> str:
    """The matrix products of one prompt step, each timed alone (twenty launches back to back, and one
    launch after L2 was overwritten), with their share of ``peak_tflops``.  With a build that stamps
    times inside the CTA-pair kernel (GIBBS_B200_NVCC_FLAGS=-DGB_PAIR_TRACE) the phases of the first
    pair of one launch follow each product: microseconds after the kernel's start at which the
    producer had set up, met its dependency and issued its last load; the MMA thread saw its first
    full stage, had issued the first tile and all tiles, and how long it waited for a free
    accumulator and for full stages (after the pipeline had filled); the epilogue saw the first
    accumulator, stored the first tile, saw the last accumulator and was done, and how long it waited."""
    import ctypes
    from .. import ops
    from ..ops.library import library
    lib = library("tensorcore")
    trace = None
    if hasattr(lib, "gb_linear_pair_trace"):
        lib.gb_linear_pair_trace.argtypes = [ctypes.c_void_p]
        trace = torch.zeros(1024 * 2 * 3 * 8, dtype=torch.int64, device=device)
    h, f = cfg.hidden_size, cfg.ffn_dim
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    shapes = [("gate_up (SwiGLU)", 2 * f, h, "swiglu"), ("down (32-bit out)", h, f, "f32"),
              ("out_proj (32-bit out)", h, h, "f32"), ("in_proj", 3 * h, h, "bf16"), ("qkv", qkv, h, "bf16")]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    gen = torch.Generator(device=device).manual_seed(0)
    lines = [f"{n_tokens} tokens; of {peak_tflops:.0f} TFLOP/s"]
    for name, n, k, mode in shapes:
        a = (torch.randn(n_tokens, k, device=device, generator=gen) * 0.5).bfloat16()
        w = (torch.randn(n, k, device=device, generator=gen) * 0.02).bfloat16()
        out = torch.empty(n_tokens, n // 2 if mode == "swiglu" else n,
                          dtype=torch.float32 if mode == "f32" else torch.bfloat16, device=device)
        run = lambda: ops.linear_tc(a, w, None, out, swiglu=(mode == "swiglu"))
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(20):
            run()
        e1.record()
        torch.cuda.synchronize()
        b2b = e0.elapsed_time(e1) / 20 * 1e3
        cold = []
        for _ in range(5):
            flush.fill_(1)
            torch.cuda.synchronize()
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            cold.append(e0.elapsed_time(e1) * 1e3)
        flops = 2.0 * n_tokens * n * k
        lines.append(f"{name:22s} N={n:6d} K={k:5d}  back to back {b2b:6.1f} us = {flops / b2b / 1e6 / peak_tflops:.3f}"
                     f"   alone, cold L2 {statistics.median(cold):6.1f} us")
        if trace is not None:
            trace.zero_()
            lib.gb_linear_pair_trace(ctypes.c_void_p(trace.data_ptr()))
            run()
            torch.cuda.synchronize()
            lib.gb_linear_pair_trace(ctypes.c_void_p(0))
            P, M, E = (trace.cpu().view(1024, 2, 3, 8)[0, 0, i].tolist() for i in range(3))
            if P[0]:
                us = lambda x: (x - P[0]) / 1e3 if x else -1.0
                cyc = lambda c: c / 1.9e3                 # cycles of the SM clock -> us, roughly
                lines.append(f"    producer: set up {us(P[1]):.1f}, dependency {us(P[2]):.1f}, last load {us(P[4]):.1f}, "
                             f"kernel end {us(P[5]):.1f} | MMA: first stage {us(M[1]):.1f}, first tile issued {us(M[2]):.1f}, "
                             f"all {us(M[3]):.1f} ({M[4]} tiles), waited ~{cyc(M[5]):.1f} for accumulators, "
                             f"~{cyc(M[6]):.1f} for stages | epilogue: first accumulator {us(E[1]):.1f}, stored "
                             f"{us(E[2]):.1f}, last accumulator {us(E[3]):.1f}, done {us(E[4]):.1f}, waited ~{cyc(E[5]):.1f}")
    return "\n".join(lines)


def prompt_attention_times(lengths=(2048, 4096, 8192, 16384), shapes=((32, 8, 64), (16, 4, 128)), page_size: int = 16,
                           device="cuda:0") -> str:
    """The attention kernel of a prompt alone: one request of n tokens from position 0, pages in a
    random order, twenty launches back to back; for every (heads, kv heads, head size) and length
    the time of a launch and the rate of its products (the causal half: 2 n (n + 1) heads head_size
    flops)."""
    import types
    from .. import ops
    gen = torch.Generator(device=device).manual_seed(0)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=device)
    lines = []
    for heads, kvh, hd in shapes:
        for n in lengths:
            nb = -(-n // page_size)
            kp = (torch.randn(nb, kvh, page_size, hd, device=device, generator=gen) * 0.5).bfloat16()
            vp = torch.randn(nb, kvh, page_size, hd, device=device, generator=gen).bfloat16()
            q = (torch.randn(n, heads * hd, device=device, generator=gen) * 0.5).bfloat16()
            out = torch.empty_like(q)
            status = torch.zeros(1, dtype=torch.int32, device=device)
            table = torch.randperm(nb, device=device, generator=gen).to(torch.int32)[None, :].contiguous()
            tok_req, tok_pos = torch.zeros(n, dtype=torch.int32, device=device), torch.arange(n, dtype=torch.int32, device=device)
            step = types.SimpleNamespace(n_requests=1, q_start=i32([0]), q_len=i32([n]), start_pos=i32([0]),
                                         max_q_len=n, max_ctx_len=n)
            run = lambda: ops.paged_attention(q, heads, kvh, hd, kp, vp, table, tok_req, tok_pos, hd ** -0.5, 0, out,
                                              status, hints=step)
            for _ in range(3):
                run()
            torch.cuda.synchronize()
            e0, e1 = _events()
            e0.record()
            for _ in range(20):
                run()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 20 * 1e3
            if int(status.item()):
                raise RuntimeError(f"attention reported status {int(status.item())}")
            flops = 2.0 * n * (n + 1) * heads * hd
            lines.append(f"{heads:3d} / {kvh} heads of {hd:3d}, {n:6d} tokens: {us:8.1f} us  {flops / us / 1e6:6.0f} TFLOP/s")
    return "\n".join(lines)


def format_timeline(rows, what: str = "decode") -> str:
    short = lambda n: n.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
    span = max(r[2] + r[3] for r in rows)
    out = [f"one {what} step: {len(rows)} kernels, {span:.1f} us from the first kernel's start to the last one's end",
           "by kernel: launches, sum of durations (they overlap), sum added to the chain of dependent launches"]
    agg: dict = {}
    for name, grid, _, dur, adds in rows:
        a = agg.setdefault((short(name), grid), [0, 0.0, 0.0])
        a[0] += 1
        a[1] += dur
        a[2] += adds
    for (name, grid), (n, dur, adds) in sorted(agg.items(), key=lambda kv: -kv[1][2]):
        out.append(f"{n:4d} {dur:9.1f} us {adds:8.1f} us  {adds / n:6.1f} us each  {name} grid {grid}")
    return "\n".join(out)


def decode_kernel_trace(engine: Engine, batch: int, prompt_len: int, seed: int = 0) -> str:
    """Time stamps from inside the cluster product kernels of one decode step (needs a build with
    GIBBS_B200_NVCC_FLAGS=-DGB_DECODE_TRACE and GIBBS_B200_DECODE_ROWS >= batch): for the first CTA
    of every launch, when its phases were reached, in microseconds after the kernel's start."""
    import ctypes
    from ..ops.library import library
    lib = library("tensorcore")
    if hasattr(lib, "gb_linear_tc_trace"):
        return _product_kernel_trace(engine, batch, prompt_len, seed, lib)
    if not hasattr(lib, "gb_linear_decode_trace"):
        raise RuntimeError("build with GIBBS_B200_NVCC_FLAGS=-DGB_GEMM_TRACE (the default products) or "
                           "-DGB_DECODE_TRACE (the cluster products) to trace a decode step's products")
    one_step, close = _decode_stepper(engine, batch, prompt_len, seed)
    for _ in range(6):
        one_step()
    torch.cuda.synchronize()
    buf = torch.zeros(4096 * 48, dtype=torch.int64, device=engine.device)
    if lib.gb_linear_decode_trace(ctypes.c_void_p(buf.data_ptr())) != 0:
        raise RuntimeError("gb_linear_decode_trace failed")
    one_step()
    torch.cuda.synchronize()
    lib.gb_linear_decode_trace(ctypes.c_void_p(0))
    close()
    t = buf.cpu().numpy().reshape(4096, 3, 16)
    n = int((t[:, 0, 0] != 0).sum())
    order = np.argsort(t[:n, 0, 0])
    lines = ["grid*1000+ranks, 10*normed+mode | start | TMA thread: first weights out, dependency met, last load out | "
             "MMA thread: all issued | producer/epilogue thread: dependency met, scales, first group, all groups, "
             "accumulator ready | slices sent, cluster barrier passed, end | what the kernel adds to the chain (us)"]
    base = prev_end = t[order[0], 0, 0] if n else 0
    for i in order:
        a = t[i]
        s0 = a[0, 0]
        rel = lambda v: (v - s0) / 1e3 if v else -1.0
        end = max(a[0, 8], a[1, 8], a[2, 8])
        lines.append(f"{a[0, 14]:7d} {a[0, 15]:3d} | {(s0 - base) / 1e3:8.1f} | {rel(a[0, 1]):5.1f} {rel(a[0, 2]):5.1f} "
                     f"{rel(a[0, 3]):5.1f} | {rel(a[1, 2]):5.1f} | {rel(a[2, 1]):5.1f} {rel(a[2, 2]):5.1f} "
                     f"{rel(a[2, 3]):5.1f} {rel(a[2, 4]):5.1f} {rel(a[2, 5]):5.1f} | {rel(a[2, 6]):5.1f} "
                     f"{rel(a[2, 7]):5.1f} {rel(end):5.1f} | {(end - prev_end) / 1e3:5.1f}")
        prev_end = max(prev_end, end)
    return "\n".join(lines)


def _product_kernel_trace(engine: Engine, batch: int, prompt_len: int, seed: int, lib) -> str:
    """Time stamps from inside ``gemm_tc_kernel`` (a -DGB_GEMM_TRACE build): for the first CTA of every
    product of one replayed decode step, microseconds after the CTA's start."""
    import ctypes
    lib.gb_linear_tc_trace.argtypes = [ctypes.c_void_p]
    one_step, close = _decode_stepper(engine, batch, prompt_len, seed)
    for _ in range(6):
        one_step()
    torch.cuda.synchronize()
    buf = torch.zeros(4096 * 48, dtype=torch.int64, device=engine.device)
    if lib.gb_linear_tc_trace(ctypes.c_void_p(buf.data_ptr())) != 0:
        raise RuntimeError("gb_linear_tc_trace failed")
    one_step()
    torch.cuda.synchronize()
    lib.gb_linear_tc_trace(ctypes.c_void_p(0))
    close()
    t = buf.cpu().numpy().reshape(4096, 3, 16)
    n = int((t[:, 0, 0] != 0).sum())
    order = np.argsort(t[:n, 0, 0])
    base = t[order[0], 0, 0] if n else 0
    lines = ["tiles*1000+splits, mode (0 bf16, 1 f32, 2 residual, 3 SwiGLU) | start | producer: weights out, dependency "
             "met, activations out, last load out | MMA thread: first stage full, the ring's first round consumed, all "
             "issued | epilogue: dependency met, accumulator ready, stored, end | end - dependency (us)"]
    for i in order:
        a = t[i]
        s0 = a[0, 0]
        rel = lambda v: (v - s0) / 1e3 if v else -1.0
        lines.append(f"{a[0, 14]:7d} {a[0, 15]:2d} | {(s0 - base) / 1e3:7.1f} | {rel(a[0, 1]):5.1f} {rel(a[0, 2]):5.1f} "
                     f"{rel(a[0, 3]):5.1f} {rel(a[0, 4]):5.1f} | {rel(a[1, 1]):5.1f} {rel(a[1, 2]):5.1f} {rel(a[1, 3]):5.1f} | "
                     f"{rel(a[2, 1]):5.1f} {rel(a[2, 2]):5.1f} {rel(a[2, 3]):5.1f} {rel(a[2, 8]):5.1f} | "
                     f"{(a[2, 8] - a[0, 2]) / 1e3:5.1f}")
    return "\n".join(lines)


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
