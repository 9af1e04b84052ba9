"""Trace replay: feeds given token ids through the engine step by step and
writes the logits at the wanted places.  It samples nothing and has no model
code of its own: it calls ``Engine.step``, which generation calls too.

A trace is one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits
as little-endian float32 [wanted, vocab], in the order of the entries and of
``want``.  After every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np

from .loading import load_model
from .step import Engine, StepEntry


def replay(model_dir, dtype: str, out_dir, max_tokens: int, lines=None, page_size: int = 16,
           max_live: int = 4, device: str = "cuda:0", echo=None) -> int:
    """Run a trace read from ``lines`` (default: standard input)."""
    lines = sys.stdin if lines is None else lines
    echo = sys.stdout if echo is None else echo
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = load_model(model_dir, dtype=dtype, device=device)
    capacity = -(-max(int(max_tokens), 1) // 64) * 64
    engine = Engine(model, n_pages=-(-capacity // page_size), page_size=page_size, max_requests=max_live,
                    max_step_tokens=capacity, max_context=capacity)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for ent in rec.get("entries", []):
            if not engine.is_live(ent["id"]):
                engine.open(ent["id"])
            entries.append(StepEntry(ent["id"], ent["tokens"], ent.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits is not None:
                arr = logits.detach().cpu().numpy().astype("<f4", copy=False)
                arr.tofile(out_dir / f"{rec['step']}.f32")
            engine.check_status()
        for rid in rec.get("end", []):
            if engine.is_live(rid):
                engine.close(rid)
        print(f"done {rec['step']}", file=echo, flush=True)
    return 0


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=4, help="most requests live at a time")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)
    return replay(a.model, a.dtype, a.out, a.max_tokens, page_size=a.page_size, max_live=a.max_live,
                  device=a.device)


if __name__ == "__main__":
    sys.exit(main())
