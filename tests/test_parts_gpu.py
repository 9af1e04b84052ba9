"""Each part alone against the plain function of the same part; models put
together from a hand-written plan (a layer run twice, a layer that reads
another layer's cache, a windowed layer); and a toy mixer with state of its
own that is defined here, registered, built and stepped without any change
to the framework."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from helpers import TOL, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rt(dtype):
    from gibbs_b200.parts import Runtime
    return Runtime(torch.bfloat16 if dtype == "bfloat16" else torch.float32, torch.device(DEV))


def _step_for(part_needs, before, q_lens, dtype, page_size=8, seed=0):
    """A cache manager for one mixer and a step over requests that already hold
    ``before`` positions and bring ``q_lens`` new ones."""
    from gibbs_b200.cache import CacheManager
    from gibbs_b200.engine.step import StepBuilder, StepEntry
    total = sum(a + b for a, b in zip(before, q_lens))
    cache = CacheManager([(part_needs, None)], n_pages=total // page_size + len(before) + 2, page_size=page_size,
                         n_slots=len(before), dtype=_rt(dtype).dtype, device=DEV, max_context=512)
    builder = StepBuilder(cache, DEV, max_requests=len(before), max_step_tokens=1024)
    rcs = [cache.open(i) for i in range(len(before))]
    return cache, builder, rcs


def _run_mixer(mixer, tokens_h, cuts, dtype, hidden):
    """Feed each request's rows of ``tokens_h`` ([n_r, hidden] float64 per
    request) through the mixer in the portions ``cuts`` gives; returns what
    the mixer added to a zero residual, per request."""
    from gibbs_b200.engine.step import StepEntry
    from gibbs_b200.parts import Residual
    rt = _rt(dtype)
    cache, builder, rcs = _step_for(mixer.cache_needs(), [0] * len(tokens_h), [len(t) for t in tokens_h], dtype)
    outs = [[] for _ in tokens_h]
    pos = [0] * len(tokens_h)
    for step_cut in cuts:                                    # step_cut: {request: n tokens}
        entries, rows = [], []
        for r, n in step_cut.items():
            entries.append(StepEntry(r, [0] * n, []))
            rows.append(tokens_h[r][pos[r]:pos[r] + n])
        live = [rcs[e.request_id] for e in entries]
        for e, rc in zip(entries, live):
            cache.reserve(rc, rc.length + len(e.tokens))
        step, caches = builder.build(entries, live)
        h = torch.cat(rows).to(rt.dtype).to(DEV)
        res = Residual(torch.zeros(h.shape[0], hidden, dtype=torch.float32, device=DEV))
        mixer.forward(h, res, step, caches[0])
        got = res.tensor().cpu().double()
        o = 0
        for e, rc in zip(entries, live):
            n = len(e.tokens)
            outs[e.request_id].append(got[o:o + n])
            o += n
            pos[e.request_id] += n
            cache.advance(rc, rc.length + n)
    assert int(builder.status.item()) == 0
    return [torch.cat(o) for o in outs]


CUTS = [
    [{0: 37, 1: 5, 2: 60}],                                                       # whole
    [{0: 30, 2: 2}, {0: 1, 1: 2, 2: 40}, {0: 1, 1: 3}, {0: 5, 2: 17}, {2: 1}],     # portions beside single tokens
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_alone(dtype):
    from gibbs_b200.config import PartSpec
    from gibbs_b200.parts import part_class
    torch.manual_seed(0)
    hidden, heads, kvh, hd, eps = 80, 6, 2, 16, 1e-6
    sizes = dict(hidden=hidden, heads=heads, kv_heads=kvh, head_dim=hd, eps=eps, theta=5e5)
    w = {"q_proj.weight": torch.randn(heads * hd, hidden) / 9, "k_proj.weight": torch.randn(kvh * hd, hidden) / 9,
         "v_proj.weight": torch.randn(kvh * hd, hidden) / 9, "out_proj.weight": torch.randn(hidden, heads * hd) / 9,
         "q_norm.weight": 1 + 0.2 * torch.randn(hd), "k_norm.weight": 1 + 0.2 * torch.randn(hd),
         "q_proj.bias": torch.randn(heads * hd) / 5, "k_proj.bias": torch.randn(kvh * hd) / 5,
         "v_proj.bias": torch.randn(kvh * hd) / 5, "out_proj.bias": torch.randn(hidden) / 5}
    rt = _rt(dtype)
    if dtype == "bfloat16":
        w = {k: (v.to(torch.bfloat16) if v.dim() == 2 else v) for k, v in w.items()}
    params = {"hidden": hidden, "heads": heads, "kv_heads": kvh, "head_dim": hd, "bias": True, "qk_norm": True,
              "qk_norm_eps": eps, "scale": 1 / math.sqrt(hd), "window": None,
              "position": PartSpec("rope_half_split", {"head_dim": hd, "rotary_dim": hd, "theta": 5e5})}
    mixer = part_class("mixer", "gqa_attention")(params, {k: v.to(DEV) for k, v in w.items()}, rt)
    toks = [torch.randn(n, hidden, dtype=torch.float64) for n in (37, 5, 60)]
    if dtype == "bfloat16":
        toks = [t.to(torch.bfloat16).double() for t in toks]
    plain_w = {"p." + k.replace("q_norm", "q_layernorm").replace("k_norm", "k_layernorm"): v.double()
               for k, v in w.items()}
    want = [plain.attention_mixer(t, plain_w, "p.", sizes, torch.arange(len(t))) for t in toks]
    for cuts in CUTS:
        got = _run_mixer(mixer, toks, cuts, dtype, hidden)
        for g, wv in zip(got, want):
            assert rel_err(g, wv.numpy()) < TOL[dtype] * (1 if dtype == "float32" else 2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel,bias", [(3, False), (5, True)])
def test_short_conv_part_alone(dtype, kernel, bias):
    from gibbs_b200.parts import part_class
    torch.manual_seed(kernel)
    hidden = 72
    w = {"in_proj.weight": torch.randn(3 * hidden, hidden) / 8, "conv.weight": torch.randn(hidden, 1, kernel) / 2,
         "out_proj.weight": torch.randn(hidden, hidden) / 8}
    if bias:
        w.update({"in_proj.bias": torch.randn(3 * hidden) / 4, "conv.bias": torch.randn(hidden) / 4,
                  "out_proj.bias": torch.randn(hidden) / 4})
    if dtype == "bfloat16":
        w = {k: (v.to(torch.bfloat16) if k.endswith("proj.weight") else v) for k, v in w.items()}
    tensors = {k: (v.reshape(hidden, kernel) if k == "conv.weight" else v).to(DEV) for k, v in w.items()}
    mixer = part_class("mixer", "gated_short_conv")({"hidden": hidden, "kernel": kernel, "bias": bias}, tensors,
                                                    _rt(dtype))
    toks = [torch.randn(n, hidden, dtype=torch.float64) for n in (37, 5, 60)]
    if dtype == "bfloat16":
        toks = [t.to(torch.bfloat16).double() for t in toks]
    plain_w = {"p." + k: v.double() for k, v in w.items()}
    want = [plain.short_conv_mixer(t, plain_w, "p.", {"hidden": hidden, "conv_k": kernel}) for t in toks]
    for cuts in CUTS:
        got = _run_mixer(mixer, toks, cuts, dtype, hidden)
        for g, wv in zip(got, want):
            assert rel_err(g, wv.numpy()) < TOL[dtype] * (1 if dtype == "float32" else 2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,bias", [(200, True), (192, False)])
def test_swiglu_part_alone(dtype, inner, bias):
    """inner = 192 takes the fused epilogue in bfloat16, 200 the separate kernel."""
    from gibbs_b200.parts import Residual, part_class
    torch.manual_seed(inner)
    hidden = 88
    w = {"gate.weight": torch.randn(inner, hidden) / 6, "up.weight": torch.randn(inner, hidden) / 6,
         "down.weight": torch.randn(hidden, inner) / 6}
    if bias:
        w.update({"gate.bias": torch.randn(inner) / 3, "up.bias": torch.randn(inner) / 3,
                  "down.bias": torch.randn(hidden) / 3})
    if dtype == "bfloat16":
        w = {k: (v.to(torch.bfloat16) if v.dim() == 2 else v) for k, v in w.items()}
    ffn = part_class("feed_forward", "swiglu")({"hidden": hidden, "inner": inner, "bias": bias},
                                               {k: v.to(DEV) for k, v in w.items()}, _rt(dtype))
    assert ffn.fused == (dtype == "bfloat16" and inner % 64 == 0)
    h = torch.randn(33, hidden, dtype=torch.float64)
    if dtype == "bfloat16":
        h = h.to(torch.bfloat16).double()
    names = {"gate": "w1", "up": "w3", "down": "w2"}
    plain_w = {"p." + names[k.split(".")[0]] + "." + k.split(".")[1]: v.double() for k, v in w.items()}
    want = plain.swiglu_ffn(h, plain_w, "p.")
    base = torch.randn(33, hidden)
    res = Residual(base.clone().to(DEV))
    ffn.forward(h.to(_rt(dtype).dtype).to(DEV), res, None)
    assert rel_err(res.tensor().cpu().double() - base.double(), want.numpy()) < TOL[dtype] * (1 if dtype == "float32" else 2)


def test_norm_and_position_parts_alone():
    from gibbs_b200.parts import part_class
    rt = _rt("float32")
    g = 1 + 0.3 * torch.randn(100)
    norm = part_class("norm", "rmsnorm")({"dim": 100, "eps": 1e-6}, {"weight": g.to(DEV)}, rt)
    x = torch.randn(7, 100) * 5
    want = plain.rms_norm(x.double(), g.double(), 1e-6)
    assert rel_err(norm.forward(x.to(DEV)).cpu(), want.numpy()) < 1e-6
    rows = torch.tensor([6, 2], dtype=torch.int32, device=DEV)
    assert rel_err(norm.forward(x.to(DEV), rows=rows).cpu(), want[[6, 2]].numpy()) < 1e-6
    for theta, hd in ((10000.0, 16), (1e6, 64), (5e5, 48)):
        rope = part_class("position", "rope_half_split")({"head_dim": hd, "rotary_dim": hd, "theta": theta}, {}, rt)
        r = rope.rotary()
        assert not r.adjacent_pairs and r.rotary_dim == hd
        assert torch.equal(r.inv_freq.cpu(), plain.rope_inv_freq(hd, theta, torch.float32))
    assert part_class("position", "rope_adjacent")({"head_dim": 8, "theta": 1e4}, {}, rt).rotary().adjacent_pairs
    assert part_class("position", "none")({}, {}, rt).rotary() is None
    with pytest.raises(KeyError, match="known"):
        part_class("mixer", "no_such_mixer")


# ---------------------------------------------------------------------------
# models from hand-written plans
# ---------------------------------------------------------------------------

class ToyDecayMixer:
    """A mixer with state of its own, written with tensor operations: per
    request a vector s (zero at the start); for every token s = a * s + W_in h,
    and the mixer adds W_out s to the residual stream."""
    category = "mixer"
    capturable = False                      # reads the step's host-side lists

    @classmethod
    def declare(cls, params):
        from gibbs_b200.parts import TensorDecl, VECTOR
        h, d = params["hidden"], params["state"]
        return {"w_in": TensorDecl.of(d, h), "w_out": TensorDecl.of(h, d), "decay": TensorDecl.of(d, role=VECTOR)}

    def __init__(self, params, tensors, rt):
        self.rt, self.d = rt, params["state"]
        self.w_in, self.w_out = tensors["w_in"].float(), tensors["w_out"].float()
        self.decay = tensors["decay"].float()

    def kernel_libraries(self):
        return ("core",)

    def cache_needs(self):
        from gibbs_b200.parts import SlotState
        return [SlotState((self.d,), torch.float32)]

    def forward(self, h, residual, step, caches):
        slot = caches[0]
        u = h.float() @ self.w_in.T
        out = torch.empty(h.shape[0], self.w_out.shape[0], device=h.device)
        for r, (start, n) in enumerate(zip(step.host_q_start, step.host_q_len)):
            s = slot.state[slot.host_slot_ids[r]].clone()
            for i in range(start, start + n):
                s = self.decay * s + u[i]
                out[i] = self.w_out @ s
            slot.state[slot.host_slot_ids[r]] = s
        residual.add_(out)


def _plain_toy(h, w_in, w_out, decay):
    s = torch.zeros(w_in.shape[0], dtype=torch.float64)
    out = []
    for i in range(h.shape[0]):
        s = decay * s + w_in @ h[i]
        out.append(w_out @ s)
    return torch.stack(out)


def _hand_plan(hidden=64, heads=4, kvh=2, hd=16, inner=128, vocab=300, eps=1e-5, window=24, state=10):
    """Layers: 0 toy mixer, 1 attention (all keys), 2 attention with a window, 3 attention without
    k/v of its own.  Order: 0, 1, 2, 1 again (its own cache), 3 reading the cache of entry 1."""
    from gibbs_b200.config import ModelPlan, OrderEntry, PartSpec, prenorm_layer

    def norm(name):
        return PartSpec("rmsnorm", {"dim": hidden, "eps": eps}, {"weight": name})

    def ffn(i):
        return PartSpec("swiglu", {"hidden": hidden, "inner": inner, "bias": False},
                        {"gate.weight": f"l{i}.g", "up.weight": f"l{i}.u", "down.weight": f"l{i}.d"})

    def attn(i, window=None, shares=False):
        t = {"q_proj.weight": f"l{i}.q", "out_proj.weight": f"l{i}.o", "q_norm.weight": f"l{i}.qn"}
        if not shares:
            t.update({"k_proj.weight": f"l{i}.k", "v_proj.weight": f"l{i}.v", "k_norm.weight": f"l{i}.kn"})
        return PartSpec("gqa_attention", {
            "hidden": hidden, "heads": heads, "kv_heads": kvh, "head_dim": hd, "bias": False, "qk_norm": True,
            "qk_norm_eps": eps, "scale": 1 / math.sqrt(hd), "window": window, "shares_kv": shares,
            "position": PartSpec("rope_half_split", {"head_dim": hd, "rotary_dim": hd, "theta": 1e4})}, t)

    toy = PartSpec("toy_decay", {"hidden": hidden, "state": state},
                   {"w_in": "l0.win", "w_out": "l0.wout", "decay": "l0.decay"})
    mixers = [toy, attn(1), attn(2, window=window), attn(3, shares=True)]
    layers = tuple(prenorm_layer(norm(f"l{i}.n1"), m, norm(f"l{i}.n2"), ffn(i)) for i, m in enumerate(mixers))
    order = (OrderEntry(0), OrderEntry(1), OrderEntry(2), OrderEntry(1), OrderEntry(3, reads_cache_of=1))
    return ModelPlan("hand-made", vocab, hidden, 512, PartSpec("token_embedding", {"vocab": vocab, "dim": hidden},
                                                                {"weight": "emb"}),
                     layers, order, norm("fn"), PartSpec("lm_head", {"vocab": vocab, "dim": hidden}, {"weight": "emb"}))


def _plain_hand_model(w, ids, hidden=64, heads=4, kvh=2, hd=16, eps=1e-5, window=24):
    """The same model written out plainly (whole sequence, no cache)."""
    n = len(ids)
    pos = torch.arange(n)
    x = w["emb"][torch.tensor(ids)]
    inv = plain.rope_inv_freq(hd, 1e4, torch.float64)

    def qkv(i, h, with_kv=True):
        q = plain.rms_norm((h @ w[f"l{i}.q"].T).reshape(n, heads, hd), w[f"l{i}.qn"], eps)
        q = plain.rope_half_split(q, pos, inv)
        if not with_kv:
            return q, None, None
        k = plain.rms_norm((h @ w[f"l{i}.k"].T).reshape(n, kvh, hd), w[f"l{i}.kn"], eps)
        return q, plain.rope_half_split(k, pos, inv), (h @ w[f"l{i}.v"].T).reshape(n, kvh, hd)

    def ffn(i, x):
        h = plain.rms_norm(x, w[f"l{i}.n2"], eps)
        g, u = h @ w[f"l{i}.g"].T, h @ w[f"l{i}.u"].T
        return x + (g / (1 + torch.exp(-g)) * u) @ w[f"l{i}.d"].T

    kv_of_entry1 = None
    for e, (layer, reads) in enumerate([(0, None), (1, None), (2, None), (1, None), (3, 1)]):
        h = plain.rms_norm(x, w[f"l{layer}.n1"], eps)
        if layer == 0:
            a = _plain_toy(h, w["l0.win"], w["l0.wout"], w["l0.decay"])
        else:
            q, k, v = qkv(layer, h, with_kv=reads is None)
            if e == 1:
                kv_of_entry1 = (k, v)
            if reads is not None:
                k, v = kv_of_entry1
            o = plain.causal_attention(q, k, v, 1 / math.sqrt(hd), window=window if layer == 2 else None)
            a = o.reshape(n, heads * hd) @ w[f"l{layer}.o"].T
        x = ffn(layer, x + a)
    return plain.rms_norm(x, w["fn"], eps) @ w["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_hand_made_model_with_toy_mixer_repeated_layer_shared_cache_and_window(dtype):
    from gibbs_b200 import Engine, register_part
    from gibbs_b200.parts import build_model
    from gibbs_b200.weights import TensorDict, expected_tensors
    from helpers import first_wrong, run_trace_on_engine, trace_mixed, trace_portions, trace_whole, random_ids
    register_part("mixer", "toy_decay", ToyDecayMixer)
    plan = _hand_plan()
    torch.manual_seed(4)
    tensors = {}
    for name, decl in expected_tensors(plan).items():
        shape = decl.shapes[0]
        if name.endswith("decay"):
            t = torch.rand(shape) * 0.5 + 0.4
        elif len(shape) == 1:
            t = 1 + 0.1 * torch.randn(shape)
        else:
            t = torch.randn(shape) * (0.3 if name == "emb" else 1.0 / math.sqrt(shape[-1]))
        tensors[name] = t.to(torch.bfloat16) if (dtype == "bfloat16" and len(shape) == 2) else t
    model = build_model(plan, TensorDict(tensors), torch.bfloat16 if dtype == "bfloat16" else torch.float32, DEV)
    needs = model.entry_needs()
    assert [len(n) for n, _ in needs] == [1, 1, 1, 1, 0] and needs[4][1] == 1
    eng = Engine(model, n_pages={None: 40, 24: 40}, page_size=8, max_requests=4, max_step_tokens=512)
    assert len(eng.cache.groups) == 2 and not eng.use_graphs                 # all keys; window of 24
    assert eng.plan is None and "ToyDecayMixer" in eng.plan_refusal          # no plan operations: forward methods run
    w64 = {k: v.double() for k, v in tensors.items()}
    reqs = {f"r{i}": random_ids(70 + i, n, 300) for i, n in enumerate([70, 33, 100, 5, 64])}
    for steps in (trace_whole(reqs), trace_portions(reqs), trace_mixed(reqs, capacity_tokens=320, seed=2)):
        got = run_trace_on_engine(eng, steps)
        for rid, ids in reqs.items():
            want = _plain_hand_model(w64, ids).numpy()
            bad = first_wrong(got[rid], want, TOL[dtype] * (1 if dtype == "float32" else 2))
            assert bad is None, f"{rid}: first wrong position {bad}"
    # the windowed group gave pages back while requests were still running
    assert eng.cache.free_pages() == [40, 40] and not eng.cache.live


# ---------------------------------------------------------------------------
# a feed-forward with routing and another position encoding, both defined here
# ---------------------------------------------------------------------------

class ToyRoutedFFN:
    """Top-1 routing among a few small experts, written with tensor operations:
    p = softmax(router h); e = argmax p; out = p[e] * W_out[e] relu(W_in[e] h)."""
    category = "feed_forward"

    @classmethod
    def declare(cls, params):
        from gibbs_b200.parts import TensorDecl
        h, f, e = params["hidden"], params["inner"], params["experts"]
        return {"router": TensorDecl.of(e, h), "w_in": TensorDecl.of(e * f, h), "w_out": TensorDecl.of(e * h, f)}

    def __init__(self, params, tensors, rt):
        self.rt = rt
        self.h, self.f, self.e = params["hidden"], params["inner"], params["experts"]
        self.router = tensors["router"].float()
        self.w_in = tensors["w_in"].float().reshape(self.e, self.f, self.h)
        self.w_out = tensors["w_out"].float().reshape(self.e, self.h, self.f)

    def kernel_libraries(self):
        return ("core",)

    def forward(self, h, residual, step):
        x = h.float()
        p = torch.softmax(x @ self.router.T, -1)                       # router logits and softmax in 32-bit
        top, choice = p.max(-1)
        hidden = torch.relu(torch.einsum("efh,nh->nef", self.w_in, x))
        every = torch.einsum("ehf,nef->neh", self.w_out, hidden)        # all experts; the toy keeps the chosen one
        picked = every[torch.arange(x.shape[0], device=x.device), choice]
        residual.add_(top[:, None] * picked)


def _toy_scaled_rope():
    from gibbs_b200.parts import PositionEncoding, Rotary

    class ToyScaledRope(PositionEncoding):
        """Half-split rotation of the first ``rotary_dim`` columns with every frequency divided by
        ``factor`` (positions stretched), the rest of the head left as it is."""

        def __init__(self, params, tensors, rt):
            super().__init__(params, tensors, rt)
            rd = int(params["rotary_dim"])
            inv = plain.rope_inv_freq(rd, float(params["theta"]), torch.float32) / float(params["factor"])
            self.inv_freq, self.rd = inv.to(rt.device), rd

        def rotary(self):
            return Rotary(self.inv_freq, self.rd, False)

    return ToyScaledRope


def _toy_plan(hidden=48, heads=3, kvh=1, hd=32, rd=16, factor=4.0, inner=64, experts=3, vocab=200, eps=1e-6):
    from gibbs_b200.config import ModelPlan, OrderEntry, PartSpec, prenorm_layer

    def norm(name):
        return PartSpec("rmsnorm", {"dim": hidden, "eps": eps}, {"weight": name})

    attn = PartSpec("gqa_attention", {
        "hidden": hidden, "heads": heads, "kv_heads": kvh, "head_dim": hd, "bias": False, "qk_norm": False,
        "scale": 1 / math.sqrt(hd), "window": None,
        "position": PartSpec("toy_scaled_rope", {"rotary_dim": rd, "theta": 1e4, "factor": factor})},
        {"q_proj.weight": "a.q", "k_proj.weight": "a.k", "v_proj.weight": "a.v", "out_proj.weight": "a.o"})
    routed = PartSpec("toy_routed", {"hidden": hidden, "inner": inner, "experts": experts},
                      {"router": "f.r", "w_in": "f.in", "w_out": "f.out"})
    conv = PartSpec("gated_short_conv", {"hidden": hidden, "kernel": 3, "bias": False},
                    {"in_proj.weight": "c.in", "conv.weight": "c.taps", "out_proj.weight": "c.out"})
    dense = PartSpec("swiglu", {"hidden": hidden, "inner": 64, "bias": False},
                     {"gate.weight": "d.g", "up.weight": "d.u", "down.weight": "d.d"})
    layers = (prenorm_layer(norm("n0"), attn, norm("n1"), routed), prenorm_layer(norm("n2"), conv, norm("n3"), dense))
    emb = PartSpec("token_embedding", {"vocab": vocab, "dim": hidden}, {"weight": "emb"})
    return ModelPlan("toy-routed", vocab, hidden, 256, emb, layers, (OrderEntry(0), OrderEntry(1)), norm("fn"),
                     PartSpec("lm_head", {"vocab": vocab, "dim": hidden}, {"weight": "head"}))


def _plain_toy_model(w, ids, hidden=48, heads=3, kvh=1, hd=32, rd=16, factor=4.0, inner=64, experts=3, eps=1e-6):
    n = len(ids)
    pos = torch.arange(n)
    x = w["emb"][torch.tensor(ids)]
    # layer 0: attention with the stretched partial rotation, then the routed feed-forward
    h = plain.rms_norm(x, w["n0"], eps)
    inv = plain.rope_inv_freq(rd, 1e4, torch.float64) / factor
    q = (h @ w["a.q"].T).reshape(n, heads, hd).clone()
    k = (h @ w["a.k"].T).reshape(n, kvh, hd).clone()
    v = (h @ w["a.v"].T).reshape(n, kvh, hd)
    q[..., :rd] = plain.rope_half_split(q[..., :rd], pos, inv)
    k[..., :rd] = plain.rope_half_split(k[..., :rd], pos, inv)
    o = plain.causal_attention(q, k, v, 1 / math.sqrt(hd))
    x = x + o.reshape(n, heads * hd) @ w["a.o"].T
    h = plain.rms_norm(x, w["n1"], eps)
    p = torch.softmax(h @ w["f.r"].T, -1)
    out = torch.zeros_like(x)
    for i in range(n):
        e = int(p[i].argmax())
        w_in = w["f.in"].reshape(experts, inner, hidden)[e]
        w_out = w["f.out"].reshape(experts, hidden, inner)[e]
        out[i] = p[i, e] * (w_out @ torch.relu(w_in @ h[i]))
    x = x + out
    # layer 1: the built-in short convolution and SwiGLU
    h = plain.rms_norm(x, w["n2"], eps)
    bcx = h @ w["c.in"].T
    b, c, xx = bcx[:, :hidden], bcx[:, hidden:2 * hidden], bcx[:, 2 * hidden:]
    x = x + (c * plain.causal_conv1d(b * xx, w["c.taps"])) @ w["c.out"].T
    h = plain.rms_norm(x, w["n3"], eps)
    g, u = h @ w["d.g"].T, h @ w["d.u"].T
    x = x + (g / (1 + torch.exp(-g)) * u) @ w["d.d"].T
    return plain.rms_norm(x, w["fn"], eps) @ w["head"].T


def test_routed_feed_forward_and_another_position_encoding_defined_in_the_test():
    """A feed-forward that routes and a position encoding of another kind are registered from
    here, built from a hand-written plan beside built-in parts and stepped in portions; nothing
    in the framework's files knows them."""
    from gibbs_b200 import Engine, register_part
    from gibbs_b200.parts import build_model
    from gibbs_b200.weights import TensorDict, expected_tensors
    from helpers import first_wrong, run_trace_on_engine, trace_portions, trace_tail_decoded, trace_whole, random_ids
    register_part("feed_forward", "toy_routed", ToyRoutedFFN)
    register_part("position", "toy_scaled_rope", _toy_scaled_rope())
    plan = _toy_plan()
    torch.manual_seed(9)
    tensors = {}
    for name, decl in expected_tensors(plan).items():
        shape = decl.shapes[0]
        if len(shape) == 1:
            tensors[name] = 1 + 0.1 * torch.randn(shape)
        elif name == "f.r":
            tensors[name] = torch.randn(shape) * 2.0          # decisive routing: no near-ties between experts
        else:
            tensors[name] = torch.randn(shape) * (0.3 if name == "emb" else 1.0 / math.sqrt(shape[-1]))
    model = build_model(plan, TensorDict(tensors), torch.float32, DEV)
    eng = Engine(model, n_pages=48, page_size=8, max_requests=4, max_step_tokens=256, use_graphs=False)
    w64 = {k: v.double() for k, v in tensors.items()}
    reqs = {f"r{i}": random_ids(30 + i, n, 200) for i, n in enumerate([50, 9, 77])}
    for steps in (trace_whole(reqs), trace_portions(reqs), trace_tail_decoded(reqs, tail=8)):
        got = run_trace_on_engine(eng, steps)
        for rid, ids in reqs.items():
            want = _plain_toy_model(w64, ids).numpy()
            bad = first_wrong(got[rid], want, 2e-5)
            assert bad is None, f"{rid}: first wrong position {bad}"
    assert not eng.cache.live


# ---------------------------------------------------------------------------
# another arrangement of a block, defined here
# ---------------------------------------------------------------------------

def _sandwich_block():
    from gibbs_b200.parts import Block, Residual

    class SandwichBlock(Block):
        """x += post(mixer(pre(x))); x += scale * ffn(pre2(x)): a norm after the mixer as well
        (MisterTK/gibbs arch/lib/transformer.json5:159-163, 'sandwich'), and a constant of the
        arrangement's own on the second branch."""
        ROLES = (("pre", "norm"), ("mixer", "mixer"), ("post", "norm"), ("pre2", "norm"), ("ffn", "feed_forward"))

        def _branch(self, x):
            return Residual(torch.zeros_like(x.tensor()))

        def forward(self, x, step, caches):
            branch = self._branch(x)
            self.mixer.forward(self.pre.forward(x), branch, step, self.caches_of("mixer", caches))
            x.add_(self.post.forward(branch))
            branch = self._branch(x)
            self.ffn.forward(self.pre2.forward(x), branch, step)
            x.add_(branch.tensor() * float(self.params["ffn_scale"]))

    return SandwichBlock


def test_block_arrangement_defined_in_the_test():
    """A block with five roles (a norm after the mixer) and a constant of its own is registered
    from here and built from a plan whose layers name their parts by role; a layer that gives
    other roles than the arrangement asks for is refused by name."""
    from gibbs_b200 import Engine, register_part
    from gibbs_b200.config import LayerSpec, ModelPlan, OrderEntry, PartSpec
    from gibbs_b200.parts import build_model
    from gibbs_b200.weights import TensorDict, expected_tensors
    from helpers import first_wrong, run_trace_on_engine, trace_portions, trace_tail_decoded, trace_whole, random_ids
    register_part("block", "toy_sandwich", _sandwich_block())
    hidden, vocab, eps, kernel, inner, scale = 40, 150, 1e-6, 3, 64, 0.5

    def norm(name):
        return PartSpec("rmsnorm", {"dim": hidden, "eps": eps}, {"weight": name})

    conv = PartSpec("gated_short_conv", {"hidden": hidden, "kernel": kernel, "bias": False},
                    {"in_proj.weight": "c.in", "conv.weight": "c.taps", "out_proj.weight": "c.out"})
    ffn = PartSpec("swiglu", {"hidden": hidden, "inner": inner, "bias": False},
                   {"gate.weight": "f.g", "up.weight": "f.u", "down.weight": "f.d"})
    layer = LayerSpec("toy_sandwich", (("pre", "norm", norm("n.pre")), ("mixer", "mixer", conv),
                                       ("post", "norm", norm("n.post")), ("pre2", "norm", norm("n.pre2")),
                                       ("ffn", "feed_forward", ffn)), {"ffn_scale": scale})
    emb = PartSpec("token_embedding", {"vocab": vocab, "dim": hidden}, {"weight": "emb"})
    head = PartSpec("lm_head", {"vocab": vocab, "dim": hidden}, {"weight": "emb"})
    plan = ModelPlan("toy-sandwich", vocab, hidden, 256, emb, (layer,), (OrderEntry(0), OrderEntry(0)), norm("fn"), head)
    assert layer.post.tensors == {"weight": "n.post"} and layer.part("mixer") is conv
    torch.manual_seed(21)
    tensors = {}
    for name, decl in expected_tensors(plan).items():
        shape = decl.shapes[0]
        tensors[name] = 1 + 0.1 * torch.randn(shape) if name.startswith(("n.", "fn")) else \
            torch.randn(shape) * (0.3 if name == "emb" else 1.0 / math.sqrt(shape[-1]))
    model = build_model(plan, TensorDict(tensors), torch.float32, DEV)
    assert [len(n) for n, _ in model.entry_needs()] == [1, 1]            # the layer runs twice, each run with its own state
    eng = Engine(model, n_pages=8, page_size=8, max_requests=3, max_step_tokens=256)
    assert eng.plan is None and "SandwichBlock" in eng.plan_refusal     # no plan operations: its forward runs

    def plain_model(ids):
        w = {k: v.double() for k, v in tensors.items()}
        x = w["emb"][torch.tensor(ids)]
        for _ in range(2):
            h = plain.rms_norm(x, w["n.pre"], eps)
            bcx = h @ w["c.in"].T
            b, c, xx = bcx[:, :hidden], bcx[:, hidden:2 * hidden], bcx[:, 2 * hidden:]
            a = (c * plain.causal_conv1d(b * xx, w["c.taps"].reshape(hidden, kernel))) @ w["c.out"].T
            x = x + plain.rms_norm(a, w["n.post"], eps)
            h = plain.rms_norm(x, w["n.pre2"], eps)
            g, u = h @ w["f.g"].T, h @ w["f.u"].T
            x = x + scale * ((g / (1 + torch.exp(-g)) * u) @ w["f.d"].T)
        return (plain.rms_norm(x, w["fn"], eps) @ w["emb"].T).numpy()

    reqs = {f"r{i}": random_ids(50 + i, n, vocab) for i, n in enumerate([40, 7, 66])}
    for steps in (trace_whole(reqs), trace_portions(reqs), trace_tail_decoded(reqs, tail=6)):
        got = run_trace_on_engine(eng, steps)
        for rid, ids in reqs.items():
            bad = first_wrong(got[rid], plain_model(ids), 2e-5)
            assert bad is None, f"{rid}: first wrong position {bad}"
    # a layer that does not give the arrangement's roles is refused, naming both lists
    wrong = LayerSpec("toy_sandwich", layer.parts[:2] + layer.parts[3:], {"ffn_scale": 1.0})
    bad_plan = ModelPlan("toy-sandwich", vocab, hidden, 256, emb, (wrong,), (OrderEntry(0),), norm("fn"), head)
    with pytest.raises(ValueError, match="is made of"):
        build_model(bad_plan, TensorDict({k: v for k, v in tensors.items() if k != "n.post"}), torch.float32, DEV)


# ---------------------------------------------------------------------------
# a mixer with a CUDA kernel of its own that joins the step plan
# ---------------------------------------------------------------------------

TOY_KERNEL_SOURCE = r'''
#include <cuda_bf16.h>
#include "gb_plan_op.h"

// One block per request: s = decay * s + W_in h_t; residual_t += W_out s, over the request's tokens in order.
template <typename T>
__global__ void toy_decay_kernel(const T* h, long long ldh, float* residual, long long ldr, const float* w_in,
                                 const float* w_out, const float* decay, float* state, long long slot_stride,
                                 const int* slot_ids, const int* q_start, const int* q_len, int hidden, int d) {
  extern __shared__ float s[];                 // [d]
  const int r = blockIdx.x;
  float* st = state + (long long)slot_ids[r] * slot_stride;
  for (int j = threadIdx.x; j < d; j += blockDim.x) s[j] = st[j];
  __syncthreads();
  for (int t = q_start[r]; t < q_start[r] + q_len[r]; ++t) {
    if (threadIdx.x < d) {
      float u = 0.f;
      for (int c = 0; c < hidden; ++c) u += w_in[threadIdx.x * hidden + c] * (float)h[t * ldh + c];
      s[threadIdx.x] = decay[threadIdx.x] * s[threadIdx.x] + u;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float y = 0.f;
      for (int j = 0; j < d; ++j) y += w_out[c * d + j] * s[j];
      residual[t * ldr + c] += y;
    }
    __syncthreads();
  }
  for (int j = threadIdx.x; j < d; j += blockDim.x) st[j] = s[j];
}

// operands: a0 h, a1 its row stride, a2 h is bfloat16 (0/1), a3 residual, a4 its row stride, a5 w_in, a6 w_out,
// a7 decay, a8 state of slot 0, a9 floats between slots, a10 slot ids, a11 first rows, a12 portion lengths,
// a13 requests, a14 hidden, a15 state size
extern "C" __attribute__((visibility("default")))
int toy_decay_op(const GbPlanCtx* ctx, const long long* a, const double* f, int flags) {
  const int requests = (int)a[13], hidden = (int)a[14], d = (int)a[15];
  if (requests <= 0) return 0;
  if (d > 128) return -1;
  if (a[2])
    toy_decay_kernel<__nv_bfloat16><<<requests, 128, d * sizeof(float), ctx->stream>>>(
        (const __nv_bfloat16*)a[0], a[1], (float*)a[3], a[4], (const float*)a[5], (const float*)a[6],
        (const float*)a[7], (float*)a[8], a[9], (const int*)a[10], (const int*)a[11], (const int*)a[12], hidden, d);
  else
    toy_decay_kernel<float><<<requests, 128, d * sizeof(float), ctx->stream>>>(
        (const float*)a[0], a[1], (float*)a[3], a[4], (const float*)a[5], (const float*)a[6], (const float*)a[7],
        (float*)a[8], a[9], (const int*)a[10], (const int*)a[11], (const int*)a[12], hidden, d);
  return cudaGetLastError() == cudaSuccess ? 1 : -2;
}
'''


def _toy_kernel_library(tmp_path):
    """Compile the toy kernel with nvcc against the package's public header; returns the ctypes library."""
    import ctypes
    import subprocess
    from gibbs_b200.csrc import build
    src = tmp_path / "toy_decay.cu"
    src.write_text(TOY_KERNEL_SOURCE)
    so = tmp_path / "libtoy_decay.so"
    subprocess.run([build.find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-shared", "-Xcompiler",
                    "-fPIC", "-I", str(build.HERE), str(src), "-o", str(so)], check=True)
    return ctypes.CDLL(str(so))


def _kernel_backed_toy_mixer(lib):
    import ctypes
    from gibbs_b200.engine import plan as step_plan
    from gibbs_b200.parts import Mixer, SlotState, TensorDecl, VECTOR

    class ToyKernelMixer(Mixer):
        """The toy recurrent mixer on a CUDA kernel of its own.  ``forward`` calls the kernel's
        operation function directly; ``plan_ops`` emits the same call as a record of the step plan
        under the id the walker gave the function.  Both are graph-capturable: nothing reads the host."""
        op_id = step_plan.register_op("toy_decay", lib.toy_decay_op)

        @classmethod
        def declare(cls, params):
            h, d = params["hidden"], params["state"]
            return {"w_in": TensorDecl.of(d, h, role=VECTOR), "w_out": TensorDecl.of(h, d, role=VECTOR),
                    "decay": TensorDecl.of(d, role=VECTOR)}

        def __init__(self, params, tensors, rt):
            super().__init__(params, tensors, rt)
            self.hidden, self.d = params["hidden"], params["state"]
            self.w_in, self.w_out, self.decay = (tensors[k].float().contiguous() for k in ("w_in", "w_out", "decay"))

        def cache_needs(self):
            return [SlotState((self.d,), torch.float32)]

        def _operands(self, h_ptr, h_ld, h_bf16, res_ptr, res_ld, state, slot_ids, q_start, q_len, n_req):
            return [h_ptr, h_ld, int(h_bf16), res_ptr, res_ld, self.w_in.data_ptr(), self.w_out.data_ptr(),
                    self.decay.data_ptr(), state.data_ptr(), state.stride(0), slot_ids, q_start, q_len, n_req,
                    self.hidden, self.d]

        def forward(self, h, residual, step, caches):
            class Ctx(ctypes.Structure):
                _fields_ = [("stream", ctypes.c_void_p), ("status", ctypes.c_void_p), ("sym", ctypes.c_void_p),
                            ("n_sym", ctypes.c_int)]
            slot, x = caches[0], residual.tensor()
            a = (ctypes.c_longlong * 24)(*self._operands(
                h.data_ptr(), h.stride(0), h.dtype == torch.bfloat16, x.data_ptr(), x.stride(0), slot.state,
                slot.slot_ids.data_ptr(), step.q_start.data_ptr(), step.q_len.data_ptr(), step.n_requests))
            ctx = Ctx(torch.cuda.current_stream().cuda_stream, step.status.data_ptr(), None, 0)
            assert lib.toy_decay_op(ctypes.byref(ctx), a, (ctypes.c_double * 3)(), 0) == 1

        def plan_ops(self, plan, h, caches):
            S = step_plan
            state = caches[0].state
            plan.keep(state), plan.keep(self.w_in), plan.keep(self.w_out), plan.keep(self.decay)
            plan.emit(self.op_id, self._operands(
                h.data_ptr(), h.stride(0), h.dtype == torch.bfloat16, plan.residual.data_ptr(), plan.residual.stride(0),
                state, S.sym(S.S_SLOT_IDS), S.sym(S.S_Q_START), S.sym(S.S_Q_LEN), S.sym(S.S_R)))

    return ToyKernelMixer


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_with_a_kernel_of_its_own_joins_the_step_plan(tmp_path, dtype):
    """A part outside the package compiles a kernel, registers its operation with the step walker and
    emits it from plan_ops: the model is plannable (one C call per step, CUDA graphs for decode steps)
    and nothing in the package's files names the operation.  The plan and the forward methods give
    the same bits, and both agree with the plain model."""
    from gibbs_b200 import Engine, register_part
    from gibbs_b200.parts import build_model
    from gibbs_b200.weights import TensorDict, expected_tensors
    from helpers import first_wrong, run_trace_on_engine, trace_mixed, trace_tail_decoded, trace_whole, random_ids
    register_part("mixer", "toy_decay", _kernel_backed_toy_mixer(_toy_kernel_library(tmp_path)))
    plan = _hand_plan()
    torch.manual_seed(4)
    tensors = {}
    for name, decl in expected_tensors(plan).items():
        shape = decl.shapes[0]
        if name.endswith("decay"):
            t = torch.rand(shape) * 0.5 + 0.4
        elif len(shape) == 1:
            t = 1 + 0.1 * torch.randn(shape)
        else:
            t = torch.randn(shape) * (0.3 if name == "emb" else 1.0 / math.sqrt(shape[-1]))
        tensors[name] = t.to(torch.bfloat16) if (dtype == "bfloat16" and len(shape) == 2 and ".w" not in name) else t
    model = build_model(plan, TensorDict(tensors), torch.bfloat16 if dtype == "bfloat16" else torch.float32, DEV)
    w64 = {k: v.double() for k, v in tensors.items()}
    reqs = {f"r{i}": random_ids(70 + i, n, 300) for i, n in enumerate([70, 33, 100, 5, 64])}
    got = {}
    for use_plan in (True, False):
        eng = Engine(model, n_pages={None: 40, 24: 40}, page_size=8, max_requests=4, max_step_tokens=512,
                     use_plan=use_plan)
        assert eng.use_graphs and (eng.plan is not None) == use_plan, eng.plan_refusal
        runs = [run_trace_on_engine(eng, steps) for steps in
                (trace_whole(reqs), trace_mixed(reqs, capacity_tokens=320, seed=2), trace_tail_decoded(reqs, tail=12))]
        assert eng._graphs                                   # decode steps were replayed from CUDA graphs
        got[use_plan] = runs
        for run in runs:
            for rid, ids in reqs.items():
                want = _plain_hand_model(w64, ids).numpy()
                bad = first_wrong(run[rid], want, TOL[dtype] * (1 if dtype == "float32" else 2))
                assert bad is None, f"{rid}: first wrong position {bad} (plan {use_plan})"
        assert eng.cache.free_pages() == [40, 40] and not eng.cache.live
    for a, b in zip(got[True], got[False]):
        for rid in a:
            assert np.array_equal(a[rid], b[rid]), rid


# ---------------------------------------------------------------------------
# constants another architecture would bring: a factor on the rotation, soft caps, a logit scale
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotary_factor_attention_soft_cap_and_logit_scale_are_parameters(dtype):
    """None of these is LFM2's; each is a parameter of a built-in part, given by a plan: the factor
    on the rotation's cosines and sines (position 'mscale'), a soft cap on the attention scores
    (mixer 'softcap'; the generic attention kernel applies it, the tensor-core kernels stand back),
    and the head's 'logit_scale' and 'softcap' (MisterTK/gibbs arch/lib/transformer.json5:59-75,
    170-175; src/graph/cpu.rs:674-675).  The plan walker and the forward methods agree bit for bit."""
    from gibbs_b200 import Engine
    from gibbs_b200.config import ModelPlan, OrderEntry, PartSpec, prenorm_layer
    from gibbs_b200.parts import build_model
    from gibbs_b200.weights import TensorDict, expected_tensors
    from helpers import first_wrong, run_trace_on_engine, trace_portions, trace_tail_decoded, trace_whole, random_ids
    hidden, heads, kvh, hd, rd, inner, vocab, eps = 64, 4, 2, 32, 16, 128, 260, 1e-6
    mscale, cap, logit_scale, logit_cap = 1.3, 2.0, 0.25, 5.0

    def norm(name):
        return PartSpec("rmsnorm", {"dim": hidden, "eps": eps}, {"weight": name})

    attn = PartSpec("gqa_attention", {
        "hidden": hidden, "heads": heads, "kv_heads": kvh, "head_dim": hd, "bias": False, "qk_norm": False,
        "scale": 1 / math.sqrt(hd), "window": None, "softcap": cap,
        "position": PartSpec("rope_half_split", {"head_dim": hd, "rotary_dim": rd, "theta": 1e4, "mscale": mscale})},
        {"q_proj.weight": "a.q", "k_proj.weight": "a.k", "v_proj.weight": "a.v", "out_proj.weight": "a.o"})
    ffn = PartSpec("swiglu", {"hidden": hidden, "inner": inner, "bias": False},
                   {"gate.weight": "f.g", "up.weight": "f.u", "down.weight": "f.d"})
    emb = PartSpec("token_embedding", {"vocab": vocab, "dim": hidden}, {"weight": "emb"})
    head = PartSpec("lm_head", {"vocab": vocab, "dim": hidden, "logit_scale": logit_scale, "softcap": logit_cap},
                    {"weight": "head"})
    plan = ModelPlan("toy-caps", vocab, hidden, 256, emb, (prenorm_layer(norm("n0"), attn, norm("n1"), ffn),),
                     (OrderEntry(0),), norm("fn"), head)
    torch.manual_seed(31)
    tensors = {}
    for name, decl in expected_tensors(plan).items():
        shape = decl.shapes[0]
        t = 1 + 0.1 * torch.randn(shape) if len(shape) == 1 else \
            torch.randn(shape) * (0.5 if name == "emb" else 2.0 / math.sqrt(shape[-1]))
        tensors[name] = t.to(torch.bfloat16) if (dtype == "bfloat16" and len(shape) == 2) else t
    model = build_model(plan, TensorDict(tensors), torch.bfloat16 if dtype == "bfloat16" else torch.float32, DEV)
    w = {k: v.double() for k, v in tensors.items()}

    def plain_model(ids):
        n = len(ids)
        pos = torch.arange(n)
        x = w["emb"][torch.tensor(ids)]
        h = plain.rms_norm(x, w["n0"], eps)
        q = (h @ w["a.q"].T).reshape(n, heads, hd).clone()
        k = (h @ w["a.k"].T).reshape(n, kvh, hd).clone()
        v = (h @ w["a.v"].T).reshape(n, kvh, hd)
        inv = plain.rope_inv_freq(rd, 1e4, torch.float64)
        half = rd // 2
        ang = (pos.float()[:, None] * inv.float()[None, :]).double()
        c, s = (torch.cos(ang) * mscale)[:, None, :], (torch.sin(ang) * mscale)[:, None, :]
        for t in (q, k):
            a, b = t[..., :half].clone(), t[..., half:rd].clone()
            t[..., :half], t[..., half:rd] = a * c - b * s, a * s + b * c
        out = torch.zeros(n, heads, hd, dtype=torch.float64)
        mask = pos[None, :] <= pos[:, None]
        for hh in range(heads):
            sc = (q[:, hh] @ k[:, hh // (heads // kvh)].T) / math.sqrt(hd)
            sc = cap * torch.tanh(sc / cap)
            sc = torch.where(mask, sc, torch.full_like(sc, float("-inf")))
            out[:, hh] = torch.softmax(sc, -1) @ v[:, hh // (heads // kvh)]
        x = x + out.reshape(n, heads * hd) @ w["a.o"].T
        h = plain.rms_norm(x, w["n1"], eps)
        g, u = h @ w["f.g"].T, h @ w["f.u"].T
        x = x + (g / (1 + torch.exp(-g)) * u) @ w["f.d"].T
        logits = plain.rms_norm(x, w["fn"], eps) @ w["head"].T / logit_scale
        return (logit_cap * torch.tanh(logits / logit_cap)).numpy()

    reqs = {f"r{i}": random_ids(90 + i, n, vocab) for i, n in enumerate([45, 6, 70])}
    got = {}
    for use_plan in (True, False):
        eng = Engine(model, n_pages=24, page_size=8, max_requests=3, max_step_tokens=128, use_plan=use_plan)
        assert (eng.plan is not None) == use_plan, eng.plan_refusal
        got[use_plan] = [run_trace_on_engine(eng, steps) for steps in
                         (trace_whole(reqs), trace_portions(reqs), trace_tail_decoded(reqs, tail=5))]
        for run in got[use_plan]:
            for rid, ids in reqs.items():
                want = plain_model(ids)
                assert np.abs(want).max() < logit_cap and np.abs(want).max() > 0.5 * logit_cap   # the cap bites
                bad = first_wrong(run[rid], want, TOL[dtype] * (1 if dtype == "float32" else 2))
                assert bad is None, f"{rid}: first wrong position {bad} (plan {use_plan})"
    for a, b in zip(got[True], got[False]):
        for rid in a:
            assert np.array_equal(a[rid], b[rid]), rid
    # without the factor, the cap or the scale the logits are others: the parameters are read
    plain_attn = PartSpec("gqa_attention", {**attn.params, "softcap": 0.0,
                                            "position": PartSpec("rope_half_split", {"head_dim": hd, "rotary_dim": rd, "theta": 1e4})},
                          attn.tensors)
    other = ModelPlan("toy-caps", vocab, hidden, 256, emb, (prenorm_layer(norm("n0"), plain_attn, norm("n1"), ffn),),
                      (OrderEntry(0),), norm("fn"), head)
    eng = Engine(build_model(other, TensorDict(tensors), model.rt.dtype, DEV), n_pages=24, page_size=8, max_requests=3,
                 max_step_tokens=128)
    differs = run_trace_on_engine(eng, trace_whole(reqs))
    assert rel_err(differs["r2"], got[True][0]["r2"]) > 10 * TOL[dtype]
