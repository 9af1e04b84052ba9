"""The Python entry point: a model folder in, generated token ids out.

    from gibbs_b200 import Generator, SamplingParams
    g = Generator("path/to/model", dtype="bfloat16")
    outs = g.generate([[5, 17, 42]], SamplingParams(temperature=0.0, max_new_tokens=16))

MisterTK/gibbs has no Python API; this mirrors its one-shot call
``scheduler.generate(prompt, max_new, temperature)``
(``src/scheduler/mod.rs:1080-1126``) over token ids.
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Sequence, Union

import torch

from ..parts.model import CausalLM
from ..sampling import Sampler, SamplingParams
from .loading import load_model
from .scheduler import MAX_PREFILL_CHUNK, PrefillTuner, Scheduler
from .step import Engine


DEFAULT_MAX_CONTEXT = 4096


def pages_for(model: CausalLM, page_size: int, max_running: int, ctx: int, memory_fraction: float = 0.8) -> int:
    """Pages to allocate per group: enough for ``max_running`` requests of
    ``ctx`` tokens, or what ``memory_fraction`` of the free device memory
    holds, whichever is smaller."""
    per_token = 0
    for needs, reads in model.entry_needs():
        if reads is None:
            for need in needs:
                if hasattr(need, "kv_heads"):
                    per_token += need.kv_heads * (need.head_dim + need.value_dim) \
                        * (2 if model.rt.dtype == torch.bfloat16 else 4)
    want = max_running * -(-ctx // page_size)
    if per_token == 0:
        return 1
    free, _ = torch.cuda.mem_get_info(model.rt.device)
    by_memory = int(free * memory_fraction) // (per_token * page_size)
    return max(1, min(want, by_memory))


class Generator:
    def __init__(self, model: Union[str, Path, CausalLM], dtype: str = "bfloat16", device: str = "cuda:0",
                 ctx: Optional[int] = None, page_size: int = 16, n_pages: Optional[int] = None,
                 max_running: int = 64, max_batch_tokens: int = MAX_PREFILL_CHUNK, seed: int = 0,
                 arch: Optional[str] = None, tune_prefill: bool = False):
        """``tune_prefill``: size each step's prompt budget from measured costs (the
        reference's ``PrefillTuner``) instead of the fixed ``max_batch_tokens``."""
        self.model = model if isinstance(model, CausalLM) else load_model(model, dtype=dtype, device=device, arch=arch)
        # as the reference: the context is max_position_embeddings, at most 4096, unless it is given
        # (MisterTK/gibbs arch/families/lfm2.json5:51); a checkpoint that allows 128k positions would
        # otherwise size every step's block tables, and the pools, for 128k
        ctx = int(ctx or min(self.model.plan.max_context, DEFAULT_MAX_CONTEXT))
        if n_pages is None:
            n_pages = pages_for(self.model, page_size, max_running, ctx)
        self.engine = Engine(self.model, n_pages=n_pages, page_size=page_size, max_requests=max_running,
                             max_step_tokens=max(max_batch_tokens, max_running), max_context=ctx)
        self.sampler = Sampler(self.model.rt.device)
        conf = getattr(self.model, "config", None)
        self.eos_ids = tuple(getattr(conf, "eos_token_ids", ()) or ())
        self.max_batch_tokens, self.max_running, self.seed = max_batch_tokens, max_running, seed
        self.tune_prefill = bool(tune_prefill)

    def scheduler(self, on_token=None, stop_at_eos: bool = True, overlap: bool = True) -> Scheduler:
        """``overlap``: decode steps are launched on the ids the device picked, one step
        before the host reads them (see ``engine/scheduler.py``)."""
        return Scheduler(self.engine, self.sampler, max_batch_tokens=self.max_batch_tokens,
                         max_running=self.max_running, eos_ids=self.eos_ids if stop_at_eos else (), seed=self.seed,
                         on_token=on_token, overlap=overlap, tuner=PrefillTuner() if self.tune_prefill else None)

    def generate(self, prompts: Sequence[Sequence[int]], params=None, stop_at_eos: bool = True) -> list:
        """Generated token ids for each prompt (lists of ids in, lists of ids out)."""
        single = bool(prompts) and isinstance(prompts[0], int)
        outs = self.scheduler(stop_at_eos=stop_at_eos).generate([prompts] if single else prompts, params)
        return outs[0] if single else outs
