#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM2-1.2B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

Prints ONE JSON line.  ``value`` is decoded tokens a second at the given batch
(device time over exactly K decode steps, CUDA events); ``e2e`` is the same
through the Python entry point, with token ids coming from and going to the
host every step; ``prefill`` times one whole prompt of 2,048 tokens; ``roofline``
relates the decode step to the memory bandwidth; ``points`` holds batch 1 and 64.  The region of K decode steps is timed five times
back to back; ``value`` and ``e2e`` are the median region's, with the spread
((slowest - fastest) / median) beside them.
The model has random bfloat16 weights and uniform-random token ids (there is
neither a checkpoint nor a dataset here).  Decode steps read 2.3 GB of
weights each, far more than the L2 holds, so no flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the benchmark configuration: layer sizes of the LFM2-1.2B shape
LFM2_1P2B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", hidden_size=2048, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=65536, intermediate_size=12288,
    block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256, conv_L_cache=3,
    conv_bias=False, full_attn_idxs=[2, 5, 8, 10, 12, 14], rope_theta=1000000.0, norm_eps=1e-5, tie_embedding=True,
    max_position_embeddings=4096,
)
SEED, PROMPT_LEN, CONTEXT = 2, 2048, 4096
REPEATS = 5             # regions of K decode steps timed back to back; the median is reported


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "MisterTK/gibbs is a Rust crate with Apple Metal kernels: pip cannot install it "
                      "(no setup.py or pyproject.toml), there is no cargo/rustc here, and it has no CUDA path"}))
    return 0


def other_workload(a):
    """The two other workloads this project's configurations name: mixed serving at the
    LFM2-700M shape, and a long context at the LFM2-2.6B shape."""
    import torch
    from gibbs_b200 import Generator, Lfm2Config, random_model
    from gibbs_b200.engine import benchmark as B
    base = dict(LFM2_1P2B)
    if a.workload == "serve700m":
        base.update(hidden_size=1536, num_attention_heads=24, intermediate_size=10240, max_position_embeddings=4096)
        cfg = Lfm2Config.from_dict(base)
        model = random_model(cfg, 3, dtype="bfloat16", device="cuda:0")
        gen = Generator(model, ctx=2048 + 256 + 16, page_size=16, max_running=64, max_batch_tokens=512, seed=3)
        B.measure_serving(gen, n_requests=64, min_len=16, max_len=2048, new_tokens=256, temperature=0.8, seed=1)  # warm-up
        res = B.measure_serving(gen, n_requests=64, min_len=16, max_len=2048, new_tokens=256, temperature=0.8, seed=3)
        res["workload"] = "LFM2-700M shape: 64 requests, prompts U[16, 2048], portions of 512 beside decode, 256 new tokens, T=0.8"
    elif a.workload == "sweep":
        # the benchmark's shape at other batch sizes, contexts and prompt lengths: one JSON line per point
        from gibbs_b200 import Engine
        base.update(max_position_embeddings=32768 + 256)
        model = random_model(Lfm2Config.from_dict(base), SEED, dtype="bfloat16", device="cuda:0")
        pk = B.load_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
        hbm, tensor = pk["hbm_gbs"], pk["bf16_tflops"]
        for ctx in (512, 2048, 8192, 32768):
            for batch in (1, 8, 64):
                if batch * ctx > 600_000:
                    continue
                eng = Engine(model, n_pages=batch * (ctx // 16 + 8), page_size=16, max_requests=batch,
                             max_step_tokens=2048, max_context=ctx + 128)
                d = B.measure_decode(eng, batch, ctx, 32, 4, seed=SEED)
                print(json.dumps({"decode_batch": batch, "context": d["context"], "ms_per_step": round(d["ms_per_step"], 4),
                                  "tok_s": round(d["tok_s"], 1), "gbs": round(d["gbs"], 1),
                                  "hbm_frac": round(d["gbs"] / hbm, 3)}), flush=True)
                del eng
                torch.cuda.empty_cache()
        for n in (128, 512, 2048, 8192):
            eng = Engine(model, n_pages=n // 16 + 8, page_size=16, max_requests=1, max_step_tokens=n, max_context=n + 16)
            pre = B.measure_prefill(eng, n, warmup=2, runs=3, seed=SEED)
            frac = B.prefill_flops(model, n) / (pre["ms"] / 1e3) / (tensor * 1e12)
            print(json.dumps({"prompt_tokens": n, "ms": round(pre["ms"], 3), "tok_s": round(pre["value"], 1),
                              "tensor_frac": round(frac, 3)}), flush=True)
            del eng
            torch.cuda.empty_cache()
        return 0
    else:
        base.update(num_hidden_layers=30, full_attn_idxs=[2, 6, 10, 14, 18, 22, 25, 28], intermediate_size=10752,
                    max_position_embeddings=8192)
        cfg = Lfm2Config.from_dict(base)
        model = random_model(cfg, 4, dtype="bfloat16", device="cuda:0")
        gen = Generator(model, ctx=8192, page_size=16, n_pages=64 * 80, max_running=64, max_batch_tokens=8192, seed=4)
        pre = B.measure_prefill(gen.engine, 8000, warmup=2, runs=3, seed=4)
        dec1 = B.measure_decode(gen.engine, 1, 8000, 64, 4, seed=4)
        dec64 = B.measure_decode(gen.engine, 64, 1024, 64, 4, seed=4)
        res = {"workload": "LFM2-2.6B shape (30 layers, FFN 7168): 8,000-token prompt, greedy decode at 8k, batch 64 at 1k",
               "prefill_8000_ms": round(pre["ms"], 2), "prefill_tok_s": round(pre["value"], 1),
               "decode_b1_ctx8000_tok_s": round(dec1["tok_s"], 1), "decode_b1_gbs": round(dec1["gbs"], 1),
               "decode_b64_ctx1024_tok_s": round(dec64["tok_s"], 1), "decode_b64_gbs": round(dec64["gbs"], 1)}
    print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in res.items()}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the engine's true 32-bit twin on the same (bfloat16-rounded) weights; "
                         "with --only prefill or --only decode (the benchmark line itself is bfloat16)")
    ap.add_argument("--skip-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--workload", choices=["serve700m", "long2p6b", "sweep"], default=None,
                    help="run one of the other reference workloads instead (prints its own JSON line)")
    ap.add_argument("--prompt-tokens", type=int, default=None,
                    help="with --only prefill / prefill-timeline / products: another prompt length than 2,048")
    ap.add_argument("--only", default=None,
                    choices=["decode", "prefill", "timeline", "prefill-timeline", "products", "attention", "trace"],
                    help="measure one phase only (for short profiler captures; the line is then partial); "
                         "'timeline' / 'prefill-timeline': the kernels of one decode step inside its graph / of one "
                         "prompt step, from CUPTI; 'products': the prompt step's matrix products alone (with "
                         "-DGB_PAIR_TRACE: and the phases inside the CTA-pair kernel); 'attention': the prompt attention "
                         "kernel alone at 2,048 to 16,384 tokens; 'trace': time "
                         "stamps from inside a decode step's product kernels (a -DGB_GEMM_TRACE or -DGB_DECODE_TRACE build)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    from gibbs_b200 import Generator, Lfm2Config, random_model
    from gibbs_b200.engine import benchmark as B

    if a.workload:
        return other_workload(a)
    raw = dict(LFM2_1P2B)
    full_layers = raw["num_hidden_layers"]
    if a.layers is not None and a.layers < full_layers:
        raw["num_hidden_layers"] = a.layers
        raw["full_attn_idxs"] = [i for i in raw["full_attn_idxs"] if i < a.layers]
    cfg = Lfm2Config.from_dict(raw)
    peaks = B.load_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    torch.manual_seed(0)
    if a.dtype != "bfloat16" and a.only not in ("prefill", "decode"):
        print("bench.py: --dtype float32 goes with --only prefill or --only decode")
        return 2
    prompt_tokens = PROMPT_LEN
    if a.prompt_tokens is not None:
        if a.only not in ("prefill", "prefill-timeline", "products") or not 1 <= a.prompt_tokens <= PROMPT_LEN:
            print(f"bench.py: --prompt-tokens (1 to {PROMPT_LEN}) goes with --only prefill, prefill-timeline or products")
            return 2
        prompt_tokens = a.prompt_tokens
    if a.only == "products":
        print(B.prompt_product_times(cfg, prompt_tokens, peaks["bf16_tflops"]))
        return 0
    if a.only == "attention":
        print(B.prompt_attention_times())
        return 0
    model = random_model(cfg, SEED, dtype=a.dtype, device="cuda:0", stored_dtype=torch.bfloat16)

    page_size = 16
    max_batch = max(64, a.batch)
    gen = Generator(model, ctx=CONTEXT, page_size=page_size, n_pages=max_batch * (CONTEXT // page_size),
                    max_running=max_batch, max_batch_tokens=2048)
    eng = gen.engine

    if a.only == "prefill":
        pre = B.measure_prefill(eng, prompt_tokens, warmup=a.warmup, runs=a.steps, seed=SEED)
        print(json.dumps({"partial": "prefill", "dtype": a.dtype, "prefill": pre}))
        return 0
    if a.only == "timeline":
        print(B.format_timeline(B.decode_timeline(eng, a.batch, PROMPT_LEN, seed=SEED)))
        return 0
    if a.only == "prefill-timeline":
        print(B.format_timeline(B.prefill_timeline(eng, prompt_tokens, seed=SEED), "prompt"))
        return 0
    if a.only == "trace":
        print(B.decode_kernel_trace(eng, a.batch, PROMPT_LEN, seed=SEED))
        return 0
    if a.only == "decode":
        dec = B.measure_decode(eng, a.batch, PROMPT_LEN, a.steps, a.warmup, seed=SEED)
        print(json.dumps({"partial": "decode", "dtype": a.dtype, "decode": dec}))
        return 0
    pre = B.measure_prefill(eng, PROMPT_LEN, warmup=a.warmup, runs=5, seed=SEED)
    pre_flops = B.prefill_flops(model, PROMPT_LEN)
    pre["frac"] = pre_flops / (pre["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12)

    # as many regions as the context has room for after the prompt (five by default)
    repeats = max(1, min(REPEATS, (CONTEXT - PROMPT_LEN - a.warmup - 4 * max_batch - 32) // max(a.steps, 1)))
    with B.ClockSampler() as clocks:
        dec = B.measure_decode(eng, a.batch, PROMPT_LEN, a.steps, a.warmup, seed=SEED, repeats=repeats)
    e2e = B.measure_decode_e2e(gen, a.batch, PROMPT_LEN, a.steps, a.warmup, seed=SEED, repeats=repeats)
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            if b != a.batch:
                points[f"decode_b{b}"] = round(B.measure_decode(eng, b, PROMPT_LEN, a.steps, a.warmup, seed=SEED,
                                                                 repeats=min(3, repeats))["tok_s"], 1)

    line = {
        "metric": "LFM2-1.2B decode tok/s", "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(dec["ms_per_step"], 4),
        "repeats": dec["repeats"], "spread": round(dec["spread"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) seed 2, uniform-random token ids",
        "config": {
            "model": "LFM2-1.2B shape", "global_batch": a.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "parallelism": "none (1 GPU)", "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "attention_layers": len(cfg.attention_layers), "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size, "conv_L_cache": cfg.conv_L_cache, "page_size": page_size,
            "l2": "step inputs (2.3 GB of weights) exceed L2; no flush",
        },
        "e2e": {k: (round(v, 4 if k == "spread" else 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": dec["launches"],
        "prefill": {"value": round(pre["value"], 1), "tokens": pre["tokens"], "ms": round(pre["ms"], 3),
                    "frac": round(pre["frac"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(dec["gbs"], 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(dec["gbs"] / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
