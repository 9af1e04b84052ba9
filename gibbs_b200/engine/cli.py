"""Command line in the manner of MisterTK/gibbs (``src/main.rs:20-189, 741-772``):
the options it shares with the reference keep the reference's names and
meanings (``--model``, ``--prompt``, ``--max-tokens``, ``--ctx``, ``--bench``,
``--probe-top5``, ``--arch``, ``--arch-dump``, ``--seed``); the server, TUI,
quantisation, drafting and media options of the reference have no
counterpart here.

    gibbs-b200 --model DIR --prompt-ids 5,17,42 --max-tokens 32
    gibbs-b200 --model DIR --prompt "text"        (needs DIR/tokenizer.json and the tokenizers package)
    gibbs-b200 --random CONFIG.json --seed 2 --save DIR      (write a random-weights model folder)
    gibbs-b200 --model DIR --arch-dump
    gibbs-b200 --model DIR --bench SUITE.json
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gibbs-b200", description="gibbs-b200: LFM2 inference on one B200")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--prompt", help="prompt text (needs tokenizer.json in the model folder)")
    ap.add_argument("--prompt-ids", help="prompt as comma-separated token ids")
    ap.add_argument("--max-tokens", type=int, default=None, help="most tokens to generate (default 64)")
    ap.add_argument("--ctx", type=int, default=None,
                    help="context length (default: the model's max_position_embeddings, at most 4096)")
    ap.add_argument("--temperature", type=float, default=None, help="default 0.7 for --prompt; <= 0 is greedy")
    ap.add_argument("--top-p", type=float, default=None, help="default 0.9")
    ap.add_argument("--repetition-penalty", type=float, default=1.0,
                    help="> 1: tokens among the latest 64 are made less likely (default 1.0: off)")
    ap.add_argument("--top-k", type=int, default=50, help="1..64, default 50; 0: off (the sampler's 64 candidates, narrowed by --top-p only)")
    ap.add_argument("--seed", type=int, default=None, help="sampling seed; also the seed of --random")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-batch-tokens", type=int, default=2048)
    ap.add_argument("--bench", help="suite.json: {defaults: {...}, models: [{id: DIR, ...}]}; one JSON line per model")
    ap.add_argument("--probe-top5", help="print the top-5 next-token logits (JSON) for these comma-separated ids")
    ap.add_argument("--arch", help="treat the model as this architecture, skipping detection")
    ap.add_argument("--arch-dump", action="store_true", help="print the resolved configuration and tensor map (JSON)")
    ap.add_argument("--random", help="config.json to make random weights for (with --save)")
    ap.add_argument("--save", help="folder to write the random-weights model to")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--peaks", help="JSON file with the memory bandwidth (hbm_gbs) and bf16 throughput (bf16_tflops) "
                                    "that roofline figures are related to (default: built-in figures for a B200)")
    return ap


def _ids(text: str) -> list:
    return [int(t) for t in text.replace(" ", "").split(",") if t]


def _tokenizer(folder: Path):
    path = folder / "tokenizer.json"
    if not path.exists():
        raise SystemExit(f"--prompt needs {path}; pass --prompt-ids for a model without a tokenizer")
    try:
        from tokenizers import Tokenizer
    except ImportError:
        raise SystemExit("--prompt needs the 'tokenizers' package; pass --prompt-ids instead") from None
    return Tokenizer.from_file(str(path))


def arch_dump(folder: Path, arch) -> dict:
    from ..config import parse_config
    from ..weights import Checkpoint, expected_tensors
    cfg = json.loads((folder / "config.json").read_text())
    ck = Checkpoint(folder)
    conf = parse_config(cfg, ck.names(), forced=arch)
    plan = conf.plan()
    want = expected_tensors(plan)
    return {"architecture": plan.architecture, "config": conf.dump(),
            "tensors": {n: {"expected": [list(s) for s in d.shapes], "role": d.role,
                            "found": list(ck.shape(n)) if n in ck.where else None} for n, d in want.items()},
            "unconsumed": sorted(set(ck.names()) - set(want)),
            "order": [{"layer": e.layer, "reads_cache_of": e.reads_cache_of} for e in plan.order]}


def bench_suite(path: Path, a) -> int:
    """One JSON line per model, with the reference's field names
    (``src/bench.rs:80-116``): decode_tok_s, prefill_tok_s, bytes_per_token,
    roofline_tok_s, roofline_pct, wall_ms, weights_ms, ceiling_gbps; and
    ``kernel_time_shares``, the share of a decode step's kernel time by kind of operation."""
    from . import benchmark as B
    from .api import Generator
    suite = json.loads(path.read_text())
    defaults = suite.get("defaults") or {}
    peaks = B.load_peaks(a.peaks)
    for m in suite["models"]:
        folder = Path(m["id"]) if Path(m["id"]).is_absolute() else path.parent / m["id"]
        decode_tokens = int(m.get("decode_tokens", defaults.get("decode_tokens", 128)))
        prefill_tokens = int(m.get("prefill_tokens", defaults.get("prefill_tokens", 512)))
        runs = int(m.get("runs", defaults.get("runs", 3)))
        batch = int(m.get("batch", defaults.get("batch", 1)))
        ctx = a.ctx or prefill_tokens + decode_tokens + 64
        gen = Generator(folder, dtype=a.dtype, device=a.device, ctx=ctx, page_size=a.page_size,
                        max_running=max(batch, 1), max_batch_tokens=max(a.max_batch_tokens, prefill_tokens))
        pre = B.measure_prefill(gen.engine, prefill_tokens, warmup=3, runs=runs)
        decs = [B.measure_decode(gen.engine, batch, prefill_tokens, decode_tokens, 3, seed=r) for r in range(runs)]
        dec = sorted(decs, key=lambda d: d["tok_s"])[len(decs) // 2]
        shares = B.decode_kind_shares(gen.engine, batch, prefill_tokens)
        bytes_per_token = dec["bytes_per_step"] // batch
        roof = peaks["hbm_gbs"] / (dec["bytes_per_step"] / 1e9) * batch
        print(json.dumps({
            "model": m.get("name", folder.name), "file": str(folder), "bytes_per_token": bytes_per_token,
            "bytes_basis": "streamed", "ceiling_gbps": peaks["hbm_gbs"], "decode_tok_s": round(dec["tok_s"], 1),
            "roofline_tok_s": round(roof, 1), "roofline_pct": round(100 * dec["tok_s"] / roof, 1),
            "wall_ms": round(dec["wall_ms_per_step"], 4), "gpu_ms": round(dec["ms_per_step"], 4),
            "host_ms": round(max(dec["wall_ms_per_step"] - dec["ms_per_step"], 0.0), 4),
            "dispatches": dec["launches"] / dec["steps"],
            "weights_ms": round(dec["bytes_per_step"] / (peaks["hbm_gbs"] * 1e9) * 1e3, 4),
            "prefill_tok_s": round(pre["value"], 1), "batch": batch, "kernel_time_shares": shares}), flush=True)
    return 0


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    if a.random:
        from ..config import parse_config
        from ..weights import write_random_model
        import torch
        if not a.save:
            raise SystemExit("--random needs --save DIR")
        conf = parse_config(json.loads(Path(a.random).read_text()), None, forced=a.arch)
        stored = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
        out = write_random_model(a.save, conf, a.seed or 0, dtype=stored)
        print(f"wrote {out}/config.json and {out}/model.safetensors (seed {a.seed or 0}, {a.dtype})")
        return 0
    if not a.model:
        raise SystemExit("--model DIR is required")
    folder = Path(a.model)
    if a.arch_dump:
        print(json.dumps(arch_dump(folder, a.arch), indent=1))
        return 0
    if a.bench:
        return bench_suite(Path(a.bench), a)

    from ..sampling import SamplingParams
    from .api import Generator
    from .step import StepEntry
    gen = Generator(folder, dtype=a.dtype, device=a.device, ctx=a.ctx, page_size=a.page_size, max_running=4,
                    max_batch_tokens=a.max_batch_tokens, seed=a.seed or 0, arch=a.arch)
    if a.probe_top5:
        ids = _ids(a.probe_top5)
        gen.engine.open("probe")
        logits = gen.engine.step([StepEntry("probe", ids, [len(ids) - 1])])[0]
        gen.engine.close("probe")
        row = logits.cpu().numpy()                  # the row goes to the host and is sorted there
        import numpy as np
        top = np.lexsort((np.arange(row.size), -row.astype(np.float64)))[:5]      # logit descending, id ascending
        print(json.dumps({"ids": [int(i) for i in top], "logits": [round(float(row[i]), 6) for i in top]}))
        return 0
    tok = None
    if a.prompt_ids:
        prompt = _ids(a.prompt_ids)
    elif a.prompt is not None:
        tok = _tokenizer(folder)
        prompt = tok.encode(a.prompt).ids
        print(f"Generating from prompt: {a.prompt!r}")
    else:
        raise SystemExit("give --prompt, --prompt-ids, --probe-top5, --bench or --arch-dump")
    temperature = a.temperature if a.temperature is not None else 0.7        # src/main.rs:746-749
    params = SamplingParams(temperature=temperature, top_p=a.top_p, top_k=a.top_k,
                            max_new_tokens=a.max_tokens if a.max_tokens is not None else 64, seed=a.seed,
                            repetition_penalty=a.repetition_penalty)
    import torch
    sched = gen.scheduler()
    sid = sched.submit(prompt, params)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    sched.step()                                                # prompt and first token
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    passes = 0
    while sched.has_work():
        passes += sched.step().decode[1]
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    seq = sched.sequences[sid]
    print("Output:")
    print(tok.decode(seq.output) if tok is not None else ",".join(str(t) for t in seq.output))
    print(f"Prefill: {len(prompt)} tokens in {(t1 - t0) * 1e3:.2f}ms; finish: {seq.finish.value}")
    tok_s = passes / max(t2 - t1, 1e-9)
    print(f"Decode: {passes} tokens in {(t2 - t1) * 1e3:.2f}ms ({tok_s:.1f} tok/s) on {torch.cuda.get_device_name()}")
    from . import benchmark as B
    peaks = B.load_peaks(a.peaks)
    bytes_per_token = gen.model.weight_bytes_per_step() \
        + (len(prompt) + len(seq.output)) * gen.engine.cache.kv_bytes_per_token() + gen.engine.cache.slot_bytes
    roof = peaks["hbm_gbs"] / (bytes_per_token / 1e9)
    print(f"Roofline: {100 * tok_s / roof:.1f}% of {roof:.1f} tok/s ({bytes_per_token} B/token at "
          f"{peaks['hbm_gbs']:.1f} GB/s, {peaks['source']})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
