"""The step function: one batch of (request, its next tokens) through the model.

A step takes any mix of prompt portions and single decoded tokens, cut
anywhere, runs exactly the tokens it is given as one ragged batch against the
cache that earlier steps left, and returns the 32-bit logits at the wanted
places.  The reference runs one sequence per forward call
(MisterTK/gibbs ``src/scheduler/mod.rs:1254-1530``, ``src/runtime/lm.rs:513-682``);
batching over block tables is this engine's own design.  As there, a step
continues each request exactly where it stands, and going past the context
is an error (``src/runtime/lm.rs:531-544``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache import CacheManager, OutOfPages
from ..parts.base import NotPlannable
from ..parts.model import CausalLM
from . import plan as step_plan


class StepError(RuntimeError):
    pass


@dataclass
class StepEntry:
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()          # indices into ``tokens`` whose logits are wanted


@dataclass
class StepState:
    """What the parts see of one step.  All tensors are int32 on the device."""
    n_tokens: int
    n_requests: int
    n_want: int
    token_ids: torch.Tensor           # [N]
    tok_req: torch.Tensor             # [N] index of the token's request within this step
    tok_pos: torch.Tensor             # [N] absolute position of the token in its request
    q_start: torch.Tensor             # [R] row of the request's first token in this step
    q_len: torch.Tensor               # [R] number of its tokens in this step
    start_pos: torch.Tensor           # [R] its length before this step
    ctx_len: torch.Tensor             # [R] its length after this step
    want_rows: torch.Tensor           # [W] rows whose logits are wanted
    status: torch.Tensor              # [1] set nonzero by a kernel that met a bad page id
    max_q_len: int = 0                # host copies, for launch sizing
    max_ctx_len: int = 0
    host_q_start: list = field(default_factory=list)
    host_q_len: list = field(default_factory=list)
    host_start_pos: list = field(default_factory=list)


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepBuilder:
    """Packs a step's metadata (token ids, token->request, positions, per-request
    starts and lengths, slots, wanted rows, block tables) into ONE pinned host
    buffer, copies it to the device with one transfer and hands out the views
    (``StepState`` and the cache views) the parts read.  The engine owns one;
    tests build steps for a bare cache manager with it."""

    def __init__(self, cache: CacheManager, device, max_requests: int, max_step_tokens: int, status=None):
        self.cache, self.device = cache, torch.device(device)
        self.max_requests, self.max_step_tokens = int(max_requests), int(max_step_tokens)
        n_groups = len(cache.groups)
        cap = 5 * _align4(self.max_step_tokens) + 5 * _align4(self.max_requests) \
            + n_groups * self.max_requests * cache.max_blocks + 16
        self._staging = [torch.empty(cap, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._staging_np = [t.numpy() for t in self._staging]
        self._staging_evt = [None] * 4
        self._turn = 0
        self.dev_meta = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.status = status if status is not None else ops.device_status(self.device)
        self.max_context = cache.max_context

    def build(self, entries, rcs):
        """(StepState, cache views) for entries (StepEntry) of live requests
        ``rcs``, through the builder's own device buffer."""
        n_tok = sum(len(e.tokens) for e in entries)
        n_req, n_want = len(entries), sum(len(e.want) for e in entries)
        offs, total = self._layout(n_tok, n_req, n_want)
        turn = self._fill_staging(entries, rcs, offs, n_tok, n_req, n_want)
        self.dev_meta[:total].copy_(self._staging[turn][:total], non_blocking=True)
        self._record(turn)
        return self._state(self.dev_meta, offs, entries, rcs, n_tok, n_req, n_want)

    def _layout(self, n_tok: int, n_req: int, n_want: int, fed: bool = False, mb: Optional[int] = None):
        """Offsets (in int32) of the sections of the metadata buffer, each
        16-byte aligned: token ids, token->request, token->position; per
        request first row, count, length before, length after, slot; wanted
        rows; one block table per group; and, when ``fed``, for each token the
        place among the ids picked on the device that it comes from (or -1).
        ``mb``: entries per request in a block table (default: as many as the
        context allows; a step may pack only what its longest request needs)."""
        n_groups, mb = len(self.cache.groups), (self.cache.max_blocks if mb is None else mb)
        sizes = [n_tok, n_tok, n_tok, n_req, n_req, n_req, n_req, n_req, max(n_want, 1), n_groups * n_req * mb,
                 n_tok if fed else 0]
        offs, o = [], 0
        for sz in sizes:
            offs.append(o)
            o += _align4(sz)
        return offs, o

    def _fill_staging(self, entries, rcs, offs, n_tok, n_req, n_want, fed_from=None, mb: Optional[int] = None,
                      token_arrays=None) -> int:
        """``token_arrays``: the entries' token ids as integer arrays, where the caller has made
        them already (a list of thousands of ids is converted once, not once to check and once to copy)."""
        turn = self._turn
        self._turn = (turn + 1) % len(self._staging)
        if self._staging_evt[turn] is not None:
            self._staging_evt[turn].synchronize()
        buf = self._staging_np[turn]
        ids, treq, tpos = (buf[offs[i]:offs[i] + n_tok] for i in range(3))
        qs, ql, sp, cl, sl = (buf[offs[i]:offs[i] + n_req] for i in range(3, 8))
        wr = buf[offs[8]:offs[8] + max(n_want, 1)]
        row, w_i = 0, 0
        for r, (e, rc) in enumerate(zip(entries, rcs)):
            n = len(e.tokens)
            ids[row:row + n] = e.tokens if token_arrays is None else token_arrays[r]
            treq[row:row + n] = r
            tpos[row:row + n] = np.arange(rc.length, rc.length + n, dtype=np.int32)
            qs[r], ql[r], sp[r], cl[r] = row, n, rc.length, rc.length + n
            sl[r] = rc.slot if rc.slot is not None else -1
            for w in e.want:
                wr[w_i] = row + int(w)
                w_i += 1
            row += n
        n_groups, mb = len(self.cache.groups), (self.cache.max_blocks if mb is None else mb)
        if n_groups:
            bt = buf[offs[9]:offs[9] + n_groups * n_req * mb].reshape(n_groups, n_req, mb)
            self.cache.fill_block_tables(rcs, bt)
        if fed_from is not None:
            src = buf[offs[10]:offs[10] + n_tok]
            src[:] = -1
            for r, f in enumerate(fed_from):
                if f >= 0:
                    src[qs[r]] = f
        return turn

    def _record(self, turn: int) -> None:
        evt = torch.cuda.Event()
        evt.record()
        self._staging_evt[turn] = evt

    def _state(self, dev, offs, entries, rcs, n_tok, n_req, n_want, fixed: bool = False, mb: Optional[int] = None):
        """The step's state and cache views over the device metadata buffer
        ``dev``.  ``fixed`` (graph capture): launch-sizing hints that do not
        depend on the requests' current lengths."""
        n_groups, mb = len(self.cache.groups), (self.cache.max_blocks if mb is None else mb)

        def view(i, n):
            return dev[offs[i]:offs[i] + n]

        step = StepState(
            n_tokens=n_tok, n_requests=n_req, n_want=n_want,
            token_ids=view(0, n_tok), tok_req=view(1, n_tok), tok_pos=view(2, n_tok),
            q_start=view(3, n_req), q_len=view(4, n_req), start_pos=view(5, n_req), ctx_len=view(6, n_req),
            want_rows=view(8, n_want), status=self.status,
            max_q_len=max(len(e.tokens) for e in entries),
            max_ctx_len=self.max_context if fixed else max(rc.length + len(e.tokens) for e, rc in zip(entries, rcs)),
            host_q_start=[] if fixed else [int(v) for v in np.cumsum([0] + [len(e.tokens) for e in entries[:-1]])],
            host_q_len=[] if fixed else [len(e.tokens) for e in entries],
            host_start_pos=[] if fixed else [rc.length for rc in rcs],
        )
        tables = [dev[offs[9] + g * n_req * mb: offs[9] + (g + 1) * n_req * mb].view(n_req, mb)
                  for g in range(n_groups)]
        caches = self.cache.views(tables, view(7, n_req), [] if fixed else [rc.slot for rc in rcs])
        return step, caches


class Engine:
    """A model, its cache and the step function over them."""

    def __init__(self, model: CausalLM, n_pages: int, page_size: int = 16, max_requests: int = 64,
                 max_step_tokens: int = 8192, max_context: Optional[int] = None, use_graphs: bool = True,
                 use_plan: bool = True, guard_cache: bool = False, timing: Optional[bool] = None):
        """``timing`` (default: the environment variable GIBBS_B200_TIMING=1): every operation of
        a step is timed with CUDA events and added up per kind (``timing_table``); steps then run
        without CUDA graphs and their kernels do not overlap."""
        self.model = model
        self.device = model.rt.device
        if self.device.type != "cuda":
            raise StepError("the engine runs on a CUDA device; there is no host path")
        ops.ensure_built(sorted(model.kernel_libraries()))
        self.max_context = int(max_context or model.plan.max_context)
        self.max_requests, self.max_step_tokens = int(max_requests), int(max_step_tokens)
        self.cache = CacheManager(model.entry_needs(), n_pages, page_size, self.max_requests, model.rt.dtype,
                                  self.device, self.max_context, guard=guard_cache)
        self.vocab_size = model.vocab_size
        self.status = ops.device_status(self.device)
        self.builder = StepBuilder(self.cache, self.device, self.max_requests, self.max_step_tokens, self.status)
        self.steps_run = 0
        self.fed_steps = 0          # steps some of whose tokens came from ids on the device
        # decode steps are replayed from CUDA graphs, one per batch size, unless a part of the
        # model cannot be captured (it reads host-side step data)
        self.timing = bool(os.environ.get("GIBBS_B200_TIMING", "0") == "1" if timing is None else timing)
        self.use_graphs = bool(use_graphs) and all(b.capturable for b in model.blocks) and not self.timing
        self._graphs: dict = {}
        self._graph_pool = None
        self._capture_stream = torch.cuda.Stream(device=self.device) if self.use_graphs else None
        self._graph_bufs: dict = {}
        # The host work of a step as a list of operations walked by one C call (engine/plan.py), when
        # every part of the model can be written that way; otherwise the parts' forward methods run.
        self.plan = None
        self.plan_refusal: Optional[str] = None
        if use_plan and step_plan.ENABLED:
            try:
                self.plan = step_plan.build_step_plan(model, self.cache, self.max_step_tokens, self.max_requests)
            except NotPlannable as e:
                self.plan_refusal = str(e)
        if self.timing and self.plan is not None:
            self.plan.set_timing(True)

    def timing_table(self) -> dict:
        """In timing mode: {kind of operation: (count, milliseconds)} over the steps so far
        (embed, rmsnorm, linear:<role>, short_conv, qk_rope, attention, swiglu, ...), the
        per-kernel-class table the reference prints with GIBBS_PROFILE_KERNELS=1
        (MisterTK/gibbs src/graph/metal.rs:143-148)."""
        if self.plan is None or not self.timing:
            return {}
        return self.plan.timing_table()

    # -- request life ----------------------------------------------------------
    def open(self, request_id) -> None:
        self.cache.open(request_id)

    def close(self, request_id) -> None:
        self.cache.close(request_id)

    def length(self, request_id) -> int:
        return self.cache.live[request_id].length

    def is_live(self, request_id) -> bool:
        return request_id in self.cache.live

    # -- the step ---------------------------------------------------------------
    def can_run(self, entries: Sequence[StepEntry]) -> bool:
        """Whether the pools have the pages this step would take (what the
        requests' windows have passed counts as free, as ``reserve_all`` gives
        it back first)."""
        live = self.cache.live
        return self.cache.can_reserve_all([(live[e.request_id], live[e.request_id].length + len(e.tokens))
                                           for e in entries])

    def _validate(self, entries):
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        total = 0
        arrays = []
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if e.request_id not in self.cache.live:
                raise StepError(f"request {e.request_id!r} is not open")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            if n <= 32:
                # (a decoded token or a short portion: cheaper to look at than to turn into an array)
                ids = e.tokens
                bad = [t for t in ids if not 0 <= int(t) < self.vocab_size]
            else:
                ids = np.asarray(e.tokens)
                if ids.ndim != 1 or ids.dtype.kind not in "iu":
                    raise StepError(f"request {e.request_id!r}: token ids are a flat sequence of integers")
                bad = ids[(ids < 0) | (ids >= self.vocab_size)] if int(ids.min()) < 0 or int(ids.max()) >= self.vocab_size \
                    else ()
            if len(bad):
                raise StepError(f"request {e.request_id!r}: token id {int(bad[0])} outside the vocabulary of "
                                f"{self.vocab_size}")
            arrays.append(ids)
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request_id!r}: wanted place {w} outside its {n} tokens")
            new_len = self.cache.live[e.request_id].length + n
            if new_len > self.max_context:
                raise StepError(f"request {e.request_id!r} would reach {new_len} positions; the context is "
                                f"{self.max_context}")
            total += n
        if len(entries) > self.max_requests:
            raise StepError(f"{len(entries)} requests in one step; the engine was made for {self.max_requests}")
        if total > self.max_step_tokens:
            raise StepError(f"{total} tokens in one step; the engine was made for {self.max_step_tokens}")
        return total, arrays

    def step(self, entries: Sequence[StepEntry], feed=None) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits [number of wanted places,
        vocab] on the device, in the order of the entries and of each entry's
        ``want``; None when nothing is wanted.  Raises OutOfPages, before
        anything changes, if the pools cannot hold the step.

        ``feed`` = (picked, places): ``picked`` are int32 token ids on the
        device (what a sampler wrote after an earlier step), ``places`` has
        one number per entry: the index in ``picked`` of the entry's single
        token, or -1 for an entry whose tokens are the given ones.  The host
        then need not have read the ids before it launches the step.

        A step in which every request brings exactly one token and wants its
        logits (a decode step) is replayed from a CUDA graph captured for that
        batch size; its logits live in the graph's own buffer and are
        overwritten by the next decode step of the same size."""
        entries = list(entries)
        n_tok, token_arrays = self._validate(entries)
        fed_from = None
        if feed is not None:
            picked, fed_from = feed[0], [int(f) for f in feed[1]]
            if len(fed_from) != len(entries):
                raise StepError("feed: one place per entry expected")
            for e, f in zip(entries, fed_from):
                if f >= 0 and (len(e.tokens) != 1 or f >= picked.numel()):
                    raise StepError(f"request {e.request_id!r}: a token fed from the device stands alone in its "
                                    f"entry and its place lies among the {picked.numel()} picked ids")
        rcs = [self.cache.live[e.request_id] for e in entries]
        self.cache.reserve_all([(rc, rc.length + len(e.tokens)) for e, rc in zip(entries, rcs)])
        try:
            logits = self._launch(entries, rcs, n_tok, fed_from, picked if fed_from is not None else None,
                                  token_arrays)
        except BaseException:
            # nothing was advanced: the pages taken for this step go back, and the caller sees
            # the requests as they stood before it
            for rc in rcs:
                self.cache.unreserve(rc)
            raise
        for e, rc in zip(entries, rcs):
            self.cache.advance(rc, rc.length + len(e.tokens))
        self.steps_run += 1
        return logits

    def _launch(self, entries, rcs, n_tok, fed_from, picked, token_arrays=None):
        """Metadata, transfer and kernels of one step whose pages are reserved."""
        n_req = len(entries)
        n_want = sum(len(e.want) for e in entries)
        bld = self.builder
        decode = self.use_graphs and n_tok == n_req and n_want == n_req
        # A step packs only as many block-table columns as its longest request needs; decode
        # steps, whose metadata layout is frozen into a CUDA graph, keep the context's full width.
        mb = self.cache.max_blocks if decode else \
            max(1, max(self.cache.pages_needed(rc.length + len(e.tokens)) for e, rc in zip(entries, rcs)))
        offs, total = bld._layout(n_tok, n_req, n_want, fed_from is not None, mb)
        turn = bld._fill_staging(entries, rcs, offs, n_tok, n_req, n_want, fed_from, mb, token_arrays)

        def fed(dev):
            if fed_from is not None:
                self.fed_steps += 1
                ops.feed_tokens(dev[offs[0]:offs[0] + n_tok], picked, dev[offs[10]:offs[10] + n_tok])

        if decode and n_req in self._graphs:
            g = self._graphs[n_req]
            g["meta"][:total].copy_(bld._staging[turn][:total], non_blocking=True)
            bld._record(turn)
            fed(g["meta"])
            g["graph"].replay()
            ops._launched(g["launches"])
            logits = g["logits"]
        else:
            dev = self._graph_meta(n_req, total) if decode else bld.dev_meta
            dev[:total].copy_(bld._staging[turn][:total], non_blocking=True)
            bld._record(turn)
            fed(dev)
            before = ops.launch_count()
            if self.plan is not None:
                args = (n_tok, n_req, n_want, max(len(e.tokens) for e in entries), dev.data_ptr(), offs, mb)
                max_ctx = self.max_context if decode else max(rc.length + len(e.tokens) for e, rc in zip(entries, rcs))
                with ops.launching_on():
                    logits = self._run_plan(*args, max_ctx)
                step = caches = None
            else:
                args = None
                step, caches = bld._state(dev, offs, entries, rcs, n_tok, n_req, n_want, fixed=decode, mb=mb)
                with ops.launching_on():
                    logits = self.model.forward(step, caches)
            if decode:
                # this run was the real step; capture the same work for the next steps of this size
                self._capture(n_req, dev, step, caches, ops.launch_count() - before, args)
        return logits

    def _graph_meta(self, batch: int, total: int) -> torch.Tensor:
        buf = self._graph_bufs.get(batch)
        if buf is None:
            # with room for the feedback section, whether or not the first step of this size has one
            size = self.builder._layout(batch, batch, batch, True)[1]
            buf = self._graph_bufs[batch] = torch.empty(max(size, total), dtype=torch.int32, device=self.device)
        return buf

    def _run_plan(self, n_tok, n_req, n_want, max_q_len, meta_ptr, offs, mb, max_ctx) -> Optional[torch.Tensor]:
        """One call into the step plan; the logits get a buffer of their own."""
        logits = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device) if n_want else None
        self.plan.run(n_tok, n_req, n_want, max_q_len, max_ctx, meta_ptr, offs, mb,
                      logits.data_ptr() if n_want else 0)
        return logits

    def _capture(self, batch: int, dev, step, caches, launches: int, plan_args=None) -> None:
        """Record the decode step of this batch size.  All graphs of an engine share one
        memory pool, and the capture is begun and ended by hand: the context manager of
        torch.cuda.graph collects garbage and empties the allocator's cache every time,
        which costs more than a hundred milliseconds per batch size."""
        graph = torch.cuda.CUDAGraph()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        torch.cuda.synchronize()
        side = self._capture_stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph.capture_begin(pool=self._graph_pool)
            try:
                with ops.launching_on(side):
                    if plan_args is not None:
                        logits = self._run_plan(*plan_args, self.max_context)
                    else:
                        logits = self.model.forward(step, caches)
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)
        ops._launched(-launches)        # the wrappers counted the captured launches, which did not run
        self._graphs[batch] = {"graph": graph, "meta": dev, "logits": logits, "launches": launches}

    def check_status(self) -> None:
        """Synchronise and raise if a kernel met a page id outside its pool."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            if code >= 16:
                raise StepError(f"a bounded wait inside a tensor-core kernel ran out (code {code}); "
                                "the kernel released what it held and returned, its output is invalid")
            raise StepError(f"a cache kernel met a page id outside its pool (code {code}); "
                            "the block tables and the pools disagree")
