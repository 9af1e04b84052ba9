"""Continuous batching above the step function: admit requests, cut prompts
into portions under a token budget, decode, finish and free.

Policy, after MisterTK/gibbs ``ContinuousBatchScheduler::step``
(``src/scheduler/mod.rs:1128-1580``):

* Admission is first come, first served, while a state slot and the pages of
  the first portion are free (``:1155-1221``).  ``max_new_tokens`` is clamped
  to ``ctx - prompt`` at submission (``:953-955``); an empty prompt becomes the
  single token 1 (``:1005-1008``).
* Every decoding request gets one token per step (``:1376-1528``).  What is
  left of the token budget goes to prompt portions, shortest remaining prompt
  first, while the oldest prefilling request keeps at least half of the
  budget (``:1231-1246, 1270-1284``).
* The first token is sampled from the logits of the last prompt position in
  the same step (``:1347-1372``).
* A request finishes with ``stop`` on an end-of-sequence id (the id is not
  emitted), with ``length`` at ``max_new_tokens`` or the context's end
  (``:1361-1371, 1504-1528``), with ``cancelled`` when its client gave up
  (``:1259-1262``) and with ``error`` when its step failed (``:1332-1340``).

Unlike the reference, all requests of a step run as ONE batch, and page ids
are real memory.  When the pages run out in mid-flight the reference carries
on (its ids are bookkeeping, ``:1294-1300``); here the request admitted last
is preempted: its pages and its slot are given back and it returns to the
head of the queue, to be recomputed from its prompt plus the tokens it has
already emitted (fixed-size state cannot be rewound).  Tokens that were
emitted are never emitted twice, and a request that cannot fit the pool even
alone ends with ``error``.

Token feedback (``overlap=True``).  The reference's Metal stream feeds the id
its argmax head picked to the next token's queued commands on the device, so
that the host never idles the GPU (``src/backend/metal/program.rs:458-544``).
Here a step whose every entry picks a token leaves its ids on the device and
on their way to pinned host memory; the next call launches the following
decode step on the device's ids *before* it waits for the host's copy, and
then reads, emits and finishes for the step before.  A request that ends on
an id nobody could foresee (end of sequence, a stop id) has then run one
token too far: the token is dropped and its pages go back like the others.
Ends by length are foreseen and leave the batch on time.  Whenever the next
step needs the host's decisions first (a request waits for admission, one
was cancelled, the pages would not suffice), the step in flight is read
before anything else happens, and the scheduler goes on as without overlap.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Optional, Sequence

from ..cache import OutOfPages, OutOfSlots
from ..sampling.params import SamplingParams
from .step import StepEntry

MAX_PREFILL_CHUNK = 2048        # src/scheduler/mod.rs:341
INITIAL_PREFILL_CHUNK = 64      # src/scheduler/mod.rs:345: the budget before a prefill has been timed
IDLE_STEP_S = 0.1               # src/scheduler/mod.rs:348: with nothing decoding a step's prefill takes about this long


class PrefillTuner:
    """Measured costs that size a step's prompt budget, after MisterTK/gibbs ``PrefillTuner``
    (``src/scheduler/mod.rs:350-403``): 64 tokens before any prefill has been timed; while
    requests decode, as many prompt tokens as cost about one decode round (1 until a decode
    round has been timed), so that prompts take roughly half of each step; with nothing
    decoding, as many as take about 100 ms; always within [1, 2048].  Both costs are
    exponential averages (0.75 old + 0.25 new) of what the scheduler's steps report.

    Here a step is one batch, so only steps that are all prompt or all decode tell the two
    costs apart; those are the ones recorded."""

    def __init__(self, whole_prompt: bool = False):
        self.prefill_s_per_token = 0.0
        self.decode_round_s = 0.0
        self.whole_prompt = whole_prompt        # one-shot generation: a prompt in one step

    def budget(self, decoding: bool) -> int:
        if self.whole_prompt:
            return 1 << 30
        if self.prefill_s_per_token == 0.0:
            return INITIAL_PREFILL_CHUNK
        if decoding:
            if self.decode_round_s == 0.0:
                return 1                         # decode cost not timed yet: the step goes to the decoding requests
            target = self.decode_round_s
        else:
            target = IDLE_STEP_S
        return max(1, min(MAX_PREFILL_CHUNK, int(target / self.prefill_s_per_token)))

    def record(self, prefill: tuple, decode: tuple) -> None:
        """``prefill`` = (seconds, prompt tokens), ``decode`` = (seconds, decoded tokens) of one step."""
        def ewma(old, new):
            return new if old == 0.0 else 0.75 * old + 0.25 * new
        if prefill[1] > 0 and decode[1] == 0:
            self.prefill_s_per_token = ewma(self.prefill_s_per_token, prefill[0] / prefill[1])
        elif decode[1] > 0 and prefill[1] == 0:
            self.decode_round_s = ewma(self.decode_round_s, decode[0])


class FinishReason(str, Enum):
    STOP = "stop"
    LENGTH = "length"
    ERROR = "error"
    CANCELLED = "cancelled"


class SeqState(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Sequence_:
    id: int
    prompt: list
    params: SamplingParams
    seed: int
    submitted: int                                  # submission order
    output: list = field(default_factory=list)
    fed: int = 0                                    # tokens of prompt + output already in the cache
    state: SeqState = SeqState.WAITING
    finish: Optional[FinishReason] = None
    error: Optional[str] = None
    logprobs: list = field(default_factory=list)    # a TokenLogprobInfo per emitted token, when asked for
    admitted: int = -1                              # admission order (for preemption)
    preemptions: int = 0
    cancelled: bool = False

    @property
    def tokens(self) -> list:
        return self.prompt + self.output

    def span(self, lo: int, hi: int) -> list:
        """Tokens lo..hi-1 of prompt + output, without building the whole list."""
        n = len(self.prompt)
        if hi <= n:
            return self.prompt[lo:hi]
        if lo >= n:
            return self.output[lo - n:hi - n]
        return self.prompt[lo:] + self.output[:hi - n]

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.fed

    @property
    def decoding(self) -> bool:
        """One token left to feed, and it is one this request generated."""
        return self.remaining == 1 and len(self.output) > 0


@dataclass
class StepOutput:
    """Shape of the reference's ``BatchStepOutput`` (``src/scheduler/mod.rs:539-546``)
    plus what was emitted and who finished."""
    tokens_generated: int = 0
    active_sequences: int = 0
    prefill: tuple = (0.0, 0)                       # (seconds, prompt tokens)
    decode: tuple = (0.0, 0)                        # (seconds, decoded tokens)
    emitted: list = field(default_factory=list)     # (sequence id, token)
    finished: list = field(default_factory=list)    # (sequence id, FinishReason)
    preempted: list = field(default_factory=list)   # sequence ids
    logprobs: list = field(default_factory=list)    # (sequence id, TokenLogprobInfo) of emitted tokens that asked


@dataclass
class _InFlight:
    """A launched step whose picked ids the host has not read yet."""
    seqs: list                                      # whose token it picks, in the order of the ids
    pending: object                                 # ``device_ids`` and ``wait() -> list of ids``
    launched: float
    n_prefill: int
    n_decode: int


@dataclass
class _FailedLaunch:
    """A fed step that raised: its requests end with ``error`` once the ids of
    the step before it have been read and emitted."""
    seqs: list
    error: str


class Scheduler:
    def __init__(self, engine, sampler: Callable, max_batch_tokens: int = MAX_PREFILL_CHUNK,
                 max_running: Optional[int] = None, eos_ids: Sequence[int] = (), seed: int = 0,
                 on_token: Optional[Callable] = None, overlap: bool = False,
                 tuner: Optional[PrefillTuner] = None, clock: Callable = time.perf_counter):
        """engine: ``open/close/step/can_run/max_context/max_requests``;
        sampler: ``(logits, params, seeds, counters) -> token ids``.
        ``overlap`` needs ``sampler.sample_async(...)`` (ids that stay on the
        device, with ``wait()`` for the host's copy) and an engine whose
        ``step`` takes ``feed``.  ``tuner``: a ``PrefillTuner`` sizes each step's
        prompt budget from measured costs, below ``max_batch_tokens``; without one the
        budget is ``max_batch_tokens``.  ``clock``: what steps are timed with."""
        self.engine, self.sampler = engine, sampler
        self.tuner, self.clock = tuner, clock
        self.overlap = bool(overlap)
        if self.overlap and not hasattr(sampler, "sample_async"):
            raise ValueError("overlap needs a sampler with sample_async")
        self._inflight: Optional[_InFlight] = None
        self.max_batch_tokens = max(1, int(max_batch_tokens))
        self.max_running = min(int(max_running or engine.max_requests), engine.max_requests)
        self.ctx = engine.max_context
        self.eos_ids = set(int(e) for e in eos_ids)
        self.seed = seed
        self.on_token = on_token
        self.waiting: deque = deque()
        self.running: list = []
        self.sequences: dict = {}
        self._next_id = 0
        self._admissions = 0
        self.steps = 0

    # -- submission --------------------------------------------------------------
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt] or [1]
        if len(prompt) >= self.ctx:
            raise ValueError(f"a prompt of {len(prompt)} tokens does not fit the context of {self.ctx}")
        max_new = min(params.max_new_tokens, self.ctx - len(prompt))
        if max_new != params.max_new_tokens:
            params = SamplingParams(**{**params.__dict__, "max_new_tokens": max_new})
        sid = self._next_id
        self._next_id += 1
        seed = params.seed if params.seed is not None else (self.seed * 0x9E3779B1 + sid * 0x85EBCA77 + 1)
        seq = Sequence_(sid, prompt, params, seed & ((1 << 64) - 1), submitted=sid)
        self.sequences[sid] = seq
        self.waiting.append(seq)
        return sid

    def cancel(self, sid: int) -> None:
        """The client gave up: the request ends at the next step."""
        self.sequences[sid].cancelled = True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None)

    # -- internals ---------------------------------------------------------------
    def _finish(self, seq: Sequence_, reason: FinishReason, out: StepOutput, error: Optional[str] = None):
        if seq.state == SeqState.RUNNING:
            self.engine.close(seq.id)
            self.running.remove(seq)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        seq.state, seq.finish, seq.error = SeqState.FINISHED, reason, error
        out.finished.append((seq.id, reason))

    def _preempt(self, seq: Sequence_, out: StepOutput):
        self.engine.close(seq.id)
        self.running.remove(seq)
        seq.state, seq.fed = SeqState.WAITING, 0
        seq.preemptions += 1
        self.waiting.appendleft(seq)
        out.preempted.append(seq.id)

    def _admit(self, budget: int, out: StepOutput):
        while self.waiting and len(self.running) < self.max_running:
            seq = self.waiting[0]
            if seq.cancelled:
                self._finish(seq, FinishReason.CANCELLED, out)
                continue
            try:
                self.engine.open(seq.id)
            except OutOfSlots:
                break
            first = min(seq.remaining, max(budget, 1))
            # the running requests' next tokens are counted too, so that a request is not
            # admitted only to be preempted in the same step
            others = [StepEntry(s.id, s.span(s.fed, s.fed + 1)) for s in self.running if s.remaining > 0]
            if not self.engine.can_run(others + [StepEntry(seq.id, seq.span(0, first))]):
                self.engine.close(seq.id)
                if not self.running:
                    # nothing else holds pages: this request can never start
                    self.waiting.popleft()
                    seq.state = SeqState.WAITING
                    self._finish(seq, FinishReason.ERROR, out,
                                 f"the cache pool cannot hold the first {first} tokens of this request")
                    continue
                break
            self.waiting.popleft()
            seq.state, seq.admitted = SeqState.RUNNING, self._admissions
            self._admissions += 1
            self.running.append(seq)

    def _prompt_budget(self, n_decoding: int) -> int:
        """Prompt tokens this step may take beside ``n_decoding`` decoded tokens."""
        budget = max(self.max_batch_tokens - n_decoding, 0)
        if self.tuner is not None:
            budget = min(budget, self.tuner.budget(n_decoding > 0))
        return budget

    def _plan(self) -> list:
        """(sequence, number of tokens) for this step."""
        plan = [(s, 1) for s in self.running if s.decoding]
        budget = self._prompt_budget(len(plan))
        prefilling = sorted((s for s in self.running if not s.decoding), key=lambda s: (s.remaining, s.submitted))
        if not prefilling:
            return plan
        if budget == 0 and not plan:
            budget = 1
        oldest = min(prefilling, key=lambda s: s.submitted)
        reserved = min(oldest.remaining, -(-budget // 2))
        left = budget
        for s in prefilling:
            if s is oldest:
                reserved = 0
                avail = left
            else:
                avail = max(left - reserved, 0)
            n = min(s.remaining, avail)
            if n > 0:
                plan.append((s, n))
                left -= n
        return plan

    # -- one step ----------------------------------------------------------------
    def step(self) -> StepOutput:
        out = StepOutput()
        self.steps += 1
        prev = self._inflight
        if prev is not None:
            # the next decode step goes out on the device's ids before the host reads this one's
            nxt = self._launch_fed(prev)
            self._inflight = nxt if isinstance(nxt, _InFlight) else None
            self._collect(prev, out)
            if isinstance(nxt, _FailedLaunch):
                # as a failing step ends its requests without overlap (below); a decode error
                # ends the sequences of that step only (src/scheduler/mod.rs:1491-1499)
                for seq in nxt.seqs:
                    if seq.state == SeqState.RUNNING:
                        self._finish(seq, FinishReason.ERROR, out, f"step failed: {nxt.error}")
            if self._inflight is not None and all(s.state != SeqState.RUNNING for s in self._inflight.seqs):
                self._inflight = None               # everybody in it has ended meanwhile
            for seq in [s for s in self.running if s.cancelled]:
                self._finish(seq, FinishReason.CANCELLED, out)
            out.active_sequences = len(self.running)
            return out
        for seq in [s for s in self.running if s.cancelled]:
            self._finish(seq, FinishReason.CANCELLED, out)
        decoding_now = sum(1 for s in self.running if s.decoding)
        self._admit(max(self._prompt_budget(decoding_now), 1), out)

        plan = self._plan()
        # Pages: drop the most recently admitted request until the step fits.
        while plan:
            entries = [StepEntry(s.id, s.span(s.fed, s.fed + n)) for s, n in plan]
            if self.engine.can_run(entries):
                break
            victim = max((s for s, _ in plan), key=lambda s: s.admitted)
            if len(self.running) == 1:
                self._finish(victim, FinishReason.ERROR, out,
                             "the cache pool cannot hold this request even alone")
            else:
                # preempt the request admitted last, whether or not it is in this step's plan
                victim = max(self.running, key=lambda s: s.admitted)
                self._preempt(victim, out)
            plan = [(s, n) for s, n in plan if s.state == SeqState.RUNNING]
        if not plan:
            out.active_sequences = len(self.running)
            return out

        entries, samplers = [], []
        n_prefill = n_decode = 0
        for s, n in plan:
            last = s.fed + n == len(s.prompt) + len(s.output)
            entries.append(StepEntry(s.id, s.span(s.fed, s.fed + n), [n - 1] if last else []))
            if last:
                samplers.append(s)
            if s.decoding:
                n_decode += 1
            else:
                n_prefill += n
        # ids may stay on the device when every request of the step picks one
        # (and none only ran to fill its cache, max_new_tokens == 0)
        # and nobody asks what the distribution said about its token: that is read from the logits at once)
        # (nor has a repetition penalty, which needs every token so far on the host)
        lag = self.overlap and len(samplers) == len(plan) and all(
            s.params.max_new_tokens > 0 and s.params.top_logprobs is None and not s.params.penalizes
            for s in samplers)
        t0 = self.clock()
        try:
            logits = self.engine.step(entries)
            args = (logits, [s.params for s in samplers], [s.seed for s in samplers],
                    [len(s.output) for s in samplers])
            # the latest tokens of each request, for those that penalise repetition
            # (MisterTK/gibbs src/scheduler/mod.rs:34-36, 79: the last 64 of prompt + generated)
            extra = {"recent": [s.span(max(0, len(s.prompt) + len(s.output) - 64), len(s.prompt) + len(s.output))
                                if s.params.penalizes else () for s in samplers]} \
                if any(s.params.penalizes for s in samplers) else {}
            if lag:
                pending, picked = self.sampler.sample_async(*args), []
            else:
                pending, picked = None, (self.sampler(*args, **extra) if samplers else [])
                infos = self._logprob_infos(logits, samplers, picked)
        except Exception as e:  # the step failed as a whole: its requests end with an error
            if isinstance(e, (OutOfPages, KeyboardInterrupt)):
                raise
            for s, _ in plan:
                self._finish(s, FinishReason.ERROR, out, f"step failed: {e}")
            out.active_sequences = len(self.running)
            return out
        for s, n in plan:
            s.fed += n
        if pending is not None:
            self._inflight = _InFlight(samplers, pending, t0, n_prefill, n_decode)
            out.active_sequences = len(self.running)
            return out
        self._emit(samplers, picked, out, infos)
        self._account(out, self.clock() - t0, n_prefill, n_decode)
        out.active_sequences = len(self.running)
        return out

    def _logprob_infos(self, logits, samplers, picked) -> dict:
        """{sequence id: TokenLogprobInfo} for the requests of a step that ask for it (the
        reference computes it from the same logits the token was picked from,
        src/scheduler/mod.rs:76-80, 1404)."""
        rows = [i for i, s in enumerate(samplers) if s.params.top_logprobs is not None]
        if not rows:
            return {}
        k = max(samplers[i].params.top_logprobs for i in rows)
        infos = self.sampler.logprob_info(logits, picked, k)       # every row of the step; those asked for are kept
        out = {}
        for i in rows:
            info, want = infos[i], samplers[i].params.top_logprobs
            out[samplers[i].id] = info if want == k else type(info)(
                info.chosen_id, info.chosen_prob, info.top_candidates[:want], info.entropy)
        return out

    def _emit(self, samplers, picked, out: StepOutput, infos: Optional[dict] = None) -> None:
        """What the picked ids mean for their requests: emitted, or the end."""
        for s, tok in zip(samplers, picked):
            if s.state != SeqState.RUNNING:
                continue                            # it ended while this step was in flight
            tok = int(tok)
            if s.params.max_new_tokens == 0:
                self._finish(s, FinishReason.LENGTH, out)
                continue
            if tok in self.eos_ids or tok in s.params.stop_ids:
                self._finish(s, FinishReason.STOP, out)
                continue
            s.output.append(tok)
            out.emitted.append((s.id, tok))
            if infos and s.id in infos:
                s.logprobs.append(infos[s.id])
                out.logprobs.append((s.id, infos[s.id]))
            out.tokens_generated += 1
            if self.on_token:
                self.on_token(s.id, tok)
            if len(s.prompt) + len(s.output) >= self.ctx or len(s.output) >= s.params.max_new_tokens:
                self._finish(s, FinishReason.LENGTH, out)

    def _account(self, out: StepOutput, dt: float, n_prefill: int, n_decode: int) -> None:
        total = max(n_prefill + n_decode, 1)
        out.prefill = (dt * n_prefill / total, n_prefill)
        out.decode = (dt * n_decode / total, n_decode)
        if self.tuner is not None:
            self.tuner.record(out.prefill, out.decode)

    # -- token feedback -----------------------------------------------------------
    def _collect(self, flight: _InFlight, out: StepOutput) -> None:
        """Wait for the ids of a launched step and do what they ask for."""
        self._emit(flight.seqs, flight.pending.wait(), out)
        self._account(out, self.clock() - flight.launched, flight.n_prefill, flight.n_decode)

    def _launch_fed(self, prev: _InFlight):
        """The decode step after ``prev``, launched on the ids ``prev`` left on the
        device: an ``_InFlight``; None when the host has to decide something
        first; a ``_FailedLaunch`` when the step raised.  A step that raises
        has given back the pages it took, but state of fixed size may already
        have moved, so its requests cannot simply be stepped again."""
        if self.waiting or any(s.cancelled for s in self.running):
            return None
        if sum(1 for s in prev.seqs if s.state == SeqState.RUNNING) != len(self.running):
            return None                             # somebody runs who is not in the step in flight
        seqs, places = [], []
        for i, s in enumerate(prev.seqs):
            if s.state != SeqState.RUNNING:
                continue                            # it ended on an id of the step before
            new = len(s.output) + 1                 # with the id that is on its way
            if new >= s.params.max_new_tokens or len(s.prompt) + new >= self.ctx:
                continue                            # it ends by length when that id is read
            seqs.append(s)
            places.append(i)
        if not seqs:
            return None
        entries = [StepEntry(s.id, [0], [0]) for s in seqs]
        if not self.engine.can_run(entries):
            return None                             # preemption is decided with every id known
        t0 = self.clock()
        try:
            logits = self.engine.step(entries, feed=(prev.pending.device_ids, places))
        except OutOfPages:
            return None                             # nothing changed; preemption is decided with every id known
        except Exception as e:
            return _FailedLaunch(seqs, str(e))
        for s in seqs:
            s.fed += 1                              # the engine has advanced, whatever the sampler does now
        try:
            pending = self.sampler.sample_async(logits, [s.params for s in seqs], [s.seed for s in seqs],
                                                [len(s.output) + 1 for s in seqs])
        except Exception as e:
            return _FailedLaunch(seqs, str(e))
        return _InFlight(seqs, pending, t0, 0, len(seqs))

    # -- convenience -------------------------------------------------------------
    def run(self, max_steps: Optional[int] = None) -> list:
        """Step until nothing is left; returns the StepOutputs."""
        outs = []
        while self.has_work() and (max_steps is None or len(outs) < max_steps):
            outs.append(self.step())
        return outs

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> list:
        """Submit prompts, run to the end, return each one's generated ids."""
        if params is None or isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        ids = [self.submit(p, q) for p, q in zip(prompts, params)]
        self.run()
        return [list(self.sequences[i].output) for i in ids]
