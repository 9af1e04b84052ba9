"""Per-request sampling controls.  Names, meanings and defaults follow
MisterTK/gibbs ``SamplingParams`` and its constants
(``src/scheduler/mod.rs:334-339, 405-446``; top-k 50: ``src/scheduler/mod.rs:178``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

DEFAULT_MAX_NEW_TOKENS = 64
DEFAULT_TEMPERATURE = 1.0
DEFAULT_TOP_P = 0.9
DEFAULT_TOP_K = 50
GREEDY_BELOW = 1e-4          # temperature at or below this is exact argmax (src/runtime/lm.rs:1073)
MAX_TOP_K = 64               # src/runtime/lm.rs:1161
MAX_TOP_LOGPROBS = 32


@dataclass(frozen=True)
class TokenLogprobInfo:
    """What the model's distribution said about one generated token (MisterTK/gibbs
    ``TokenLogprobInfo``, ``src/scheduler/mod.rs:417-423``): its probability under the softmax
    of the raw logits, the ``top_logprobs`` most probable tokens with theirs, and the
    distribution's entropy."""
    chosen_id: int
    chosen_prob: float
    top_candidates: tuple                    # ((token id, probability), ...), most probable first
    entropy: float


@dataclass(frozen=True)
class SamplingParams:
    temperature: Optional[float] = None      # None: DEFAULT_TEMPERATURE; <= 0 is greedy
    top_p: Optional[float] = None            # None: DEFAULT_TOP_P
    top_k: int = DEFAULT_TOP_K               # 1..64; 0: no narrower limit than the sampler's own 64 candidates
    max_new_tokens: int = DEFAULT_MAX_NEW_TOKENS
    seed: Optional[int] = None               # None: derived from the scheduler's seed and the request id
    stop_ids: tuple = ()                     # besides the model's own end-of-sequence ids
    top_logprobs: Optional[int] = None       # report each token's probability, the entropy and this many candidates
    repetition_penalty: float = 1.0          # > 1: tokens among the request's latest 64 are made less likely

    def __post_init__(self):
        if not 0 <= self.top_k <= MAX_TOP_K:
            raise ValueError(f"top_k {self.top_k} outside 0..{MAX_TOP_K} (0: off)")
        if not self.repetition_penalty >= 0.0:
            raise ValueError(f"repetition_penalty {self.repetition_penalty}")
        if self.max_new_tokens < 0:
            raise ValueError(f"max_new_tokens {self.max_new_tokens}")
        if self.top_logprobs is not None and not 1 <= self.top_logprobs <= MAX_TOP_LOGPROBS:
            raise ValueError(f"top_logprobs {self.top_logprobs} outside 1..{MAX_TOP_LOGPROBS}")

    @property
    def resolved_temperature(self) -> float:
        t = DEFAULT_TEMPERATURE if self.temperature is None else float(self.temperature)
        return max(t, 0.0)

    @property
    def penalizes(self) -> bool:
        """Whether the repetition penalty does anything (MisterTK/gibbs src/runtime/lm.rs:1074: a
        factor of 1 or less is off)."""
        return self.repetition_penalty > 1.0

    @property
    def resolved_top_k(self) -> int:
        """The number of candidates the sampling kernel keeps: top_k, or all 64 it can hold when
        top_k is 0 (then top_p alone narrows them)."""
        return self.top_k if self.top_k > 0 else MAX_TOP_K

    @property
    def resolved_top_p(self) -> float:
        return DEFAULT_TOP_P if self.top_p is None else float(self.top_p)

    @property
    def greedy(self) -> bool:
        return self.resolved_temperature <= GREEDY_BELOW
