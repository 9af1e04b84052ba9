"""An engine without a GPU for scheduler tests: the real cache manager on the
host, and logits that are a pure function of the tokens a request has been
fed, so that any rescheduling must reproduce them."""
import torch

from gibbs_b200.cache import CacheManager, OutOfPages
from gibbs_b200.parts.base import PagedKV, SlotState


def fake_next(tokens, vocab):
    h = 17
    for t in tokens:
        h = (h * 31 + int(t) + 1) % 1000003
    return h % vocab


class FakeEngine:
    def __init__(self, n_pages=64, page_size=4, max_requests=4, max_context=256, vocab=50, fail_on=None):
        self.cache = CacheManager([([PagedKV(1, 2)], None), ([SlotState((2,))], None)], n_pages, page_size,
                                  max_requests, torch.float32, "cpu", max_context)
        self.max_requests, self.max_context, self.vocab = max_requests, max_context, vocab
        self.fed = {}
        self.log = []               # per step: [(request id, number of tokens, wanted?)]
        self.events = []            # "launch", "launch fed", and "read" from LaggingSampler
        self.fail_on = fail_on      # step index at which step() raises

    def open(self, rid):
        self.cache.open(rid)
        self.fed[rid] = []

    def close(self, rid):
        self.cache.close(rid)
        del self.fed[rid]

    def can_run(self, entries):
        live = self.cache.live
        return self.cache.can_reserve_all([(live[e.request_id], live[e.request_id].length + len(e.tokens))
                                           for e in entries])

    def step(self, entries, feed=None):
        if feed is not None:
            # ids that a sampler left "on the device": the fake reads them where the real engine's kernel would
            picked, places = feed
            self.events.append("launch fed")
            entries = [type(e)(e.request_id, [picked[f]] if f >= 0 else e.tokens, e.want)
                       for e, f in zip(entries, places)]
        else:
            self.events.append("launch")
        rcs = [self.cache.live[e.request_id] for e in entries]
        self.cache.reserve_all([(rc, rc.length + len(e.tokens)) for e, rc in zip(entries, rcs)])
        if self.fail_on is not None and len(self.log) == self.fail_on:
            # as the real engine: a launch that raises gives back what the step reserved
            self.log.append("failed")
            for rc in rcs:
                self.cache.unreserve(rc)
            raise RuntimeError("injected step failure")
        rows = []
        for e in entries:
            rc = self.cache.live[e.request_id]
            self.cache.advance(rc, rc.length + len(e.tokens))
            base = len(self.fed[e.request_id])
            self.fed[e.request_id].extend(e.tokens)
            for w in e.want:
                row = torch.zeros(self.vocab)
                row[fake_next(self.fed[e.request_id][:base + w + 1], self.vocab)] = 1.0
                rows.append(row)
        self.log.append([(e.request_id, len(e.tokens), bool(e.want)) for e in entries])
        self.cache.check()
        return torch.stack(rows) if rows else None


def argmax_sampler(logits, params, seeds, counters):
    return [int(torch.argmax(r)) for r in logits]


class LaggingSampler:
    """argmax whose ids "stay on the device": ``sample_async`` hands out a list
    at once, ``wait()`` notes in the engine's event list when the host read it."""

    def __init__(self, engine):
        self.engine = engine

    def __call__(self, logits, params, seeds, counters):
        self.engine.events.append("read")
        return argmax_sampler(logits, params, seeds, counters)

    def sample_async(self, logits, params, seeds, counters):
        ids, events = argmax_sampler(logits, params, seeds, counters), self.engine.events

        class Pending:
            device_ids = ids

            def wait(self):
                events.append("read")
                return list(ids)

        return Pending()


def expected_greedy(prompt, n_new, vocab, eos=()):
    toks, out = list(prompt), []
    for _ in range(n_new):
        t = fake_next(toks, vocab)
        if t in eos:
            break
        toks.append(t)
        out.append(t)
    return out


def fake_logprob_info(logits, chosen, k):
    """Host twin of the sampler's ``logprob_info`` for the fake engine's one-hot logits."""
    from gibbs_b200.sampling import TokenLogprobInfo
    out = []
    for row, c in zip(logits, chosen):
        p = torch.softmax(row.double(), 0)
        top = torch.argsort(-p, stable=True)[:k]
        ent = float(-(p * torch.log(p)).sum())
        out.append(TokenLogprobInfo(int(c), float(p[int(c)]), tuple((int(i), float(p[i])) for i in top), ent))
    return out
