"""Sampling on the device: one launch picks a token for every wanted logits
row (greedy, or temperature with top-k and top-p; ``csrc/sampling.cu``).

Randomness is counter based: the uniform number of a draw is SplitMix64 of
(the request's seed, how many tokens it has drawn so far), so a run with a
seed repeats, whatever the batching.  (The reference hashes the recent tokens
instead, ``src/runtime/lm.rs:1125-1137``.)"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import ops
from .params import SamplingParams, TokenLogprobInfo

_MASK = (1 << 64) - 1


def uniform24(seed: int, counter: int) -> float:
    """Host twin of the kernel's generator: a multiple of 2^-24 in [0, 1)."""
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def _signed(v: int) -> int:
    v &= _MASK
    return v - (1 << 64) if v >= (1 << 63) else v


class PendingIds:
    """Token ids that were picked on the device and are on their way to the
    host: ``device_ids`` can feed the next step at once, ``wait()`` gives the
    host's copy when the transfer has ended."""

    def __init__(self, device_ids: torch.Tensor, host: torch.Tensor, event):
        self.device_ids, self._host, self._event = device_ids, host, event

    def wait(self) -> list:
        self._event.synchronize()
        return self._host.tolist()


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the sampler is a CUDA kernel; there is no host path")
        self._pinned: list = []
        self._turn = 0

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                     counters: Sequence[int], recent=None) -> PendingIds:
        """Pick on the device and start the copy to pinned host memory; nothing waits."""
        out = self.sample_device(logits, params, seeds, counters, recent)
        rows = out.numel()
        if not self._pinned or self._pinned[0].numel() < rows:
            self._pinned = [torch.empty(max(rows, 64), dtype=torch.int32).pin_memory() for _ in range(4)]
        host = self._pinned[self._turn][:rows]
        self._turn = (self._turn + 1) % len(self._pinned)
        host.copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingIds(out, host, event)

    def __call__(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                 counters: Sequence[int], recent=None) -> list[int]:
        """One token id per row of ``logits`` ([rows, vocab] float32 on the device).  ``recent``:
        for each row the request's latest tokens (prompt and generated; the last 64 count), needed
        by the rows whose parameters ask for a repetition penalty."""
        out = self.sample_device(logits, params, seeds, counters, recent)
        return out.tolist()

    def _penalized(self, logits, params, recent) -> torch.Tensor:
        """A copy of ``logits`` with the repetition penalty of the rows that ask for one applied
        (the caller's logits stay as the model gave them: reports about the distribution are made
        from those)."""
        if recent is None or len(recent) != len(params):
            raise ValueError("a repetition penalty needs every row's recent tokens")
        n = ops.RECENT_TOKENS
        ids = torch.full((len(params), n), -1, dtype=torch.int32)
        for r, (p, toks) in enumerate(zip(params, recent)):
            if p.penalizes and len(toks):
                last = list(toks)[-n:]
                ids[r, :len(last)] = torch.tensor(last, dtype=torch.int32)
        pen = torch.tensor([p.repetition_penalty if p.penalizes else 1.0 for p in params], dtype=torch.float32)
        temp = torch.tensor([0.0 if p.greedy else p.resolved_temperature for p in params], dtype=torch.float32)
        ids, pen, temp = (t.to(self.device, non_blocking=True) for t in (ids, pen, temp))
        work = logits.clone()
        return ops.repetition_penalty(work, ids, pen, temp)

    def logprob_info(self, logits: torch.Tensor, chosen: Sequence[int], k: int) -> list:
        """``TokenLogprobInfo`` of every row of ``logits`` for the ids in ``chosen`` (computed by
        a kernel, read back to the host)."""
        ids = torch.tensor([int(c) for c in chosen], dtype=torch.int32, device=self.device)
        prob, entropy, top_ids, top_probs = (t.tolist() for t in ops.logprob_info(logits, ids, k))
        return [TokenLogprobInfo(int(c), p, tuple((i, q) for i, q in zip(ti, tp) if i >= 0), e)
                for c, p, e, ti, tp in zip(chosen, prob, entropy, top_ids, top_probs)]

    def sample_device(self, logits, params, seeds, counters, recent=None) -> torch.Tensor:
        rows = logits.shape[0]
        if any(p.penalizes for p in params):
            logits = self._penalized(logits, params, recent)
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(p.greedy for p in params):
            return ops.sample(logits, out)
        host = torch.tensor(
            [[p.resolved_temperature if not p.greedy else 0.0, p.resolved_top_p] for p in params], dtype=torch.float32)
        ints = torch.tensor([[p.resolved_top_k] for p in params], dtype=torch.int32)
        longs = torch.tensor([[_signed(s), int(c)] for s, c in zip(seeds, counters)], dtype=torch.int64)
        host, ints, longs = (t.to(self.device, non_blocking=True) for t in (host, ints, longs))
        return ops.sample(logits, out, temperature=host[:, 0].contiguous(), top_k=ints[:, 0].contiguous(),
                          top_p=host[:, 1].contiguous(), seed=longs[:, 0].contiguous(),
                          counter=longs[:, 1].contiguous())
