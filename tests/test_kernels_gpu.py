"""Each CUDA kernel alone against a plain float64 reference of the same
operation written here, at sizes other than the engine's tiny models: widths
and vocabularies that are no power of two, head sizes in steps of 16, odd
numbers of heads and groups."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dt(name):
    return torch.bfloat16 if name == "bfloat16" else torch.float32


def _close(got, want, dtype, scale=None):
    got = got.detach().double().cpu()
    want = want.double()
    tol = 2e-2 if dtype == "bfloat16" else 2e-5
    err = (got - want).abs().max().item()
    ref = (scale if scale is not None else want.abs().max().item()) + 1e-30
    assert err / ref < tol, f"max abs err {err:.3g} against scale {ref:.3g}"


def _quant(t, dtype):
    """Round to the kernel's storage dtype, return (device tensor, float64 copy of the rounded values)."""
    d = t.to(_dt(dtype))
    return d.to(DEV), d.double()


# --------------------------------------------------------------------------- embed / norm / swiglu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [96, 2048, 100, 4104])     # 16-byte pieces (one or several per thread) or single values
def test_embed(dtype, dim):
    from gibbs_b200 import ops
    torch.manual_seed(0)
    table, ref = _quant(torch.randn(1000, dim), dtype)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device=DEV)
    out = torch.empty(5, dim, dtype=torch.float32, device=DEV)
    ops.embed(table, ids, out)
    assert torch.equal(out.cpu().double(), ref[ids.cpu().long()])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,eps", [(96, 1e-6), (2048, 1e-5), (1000, 1e-5), (7, 1e-3)])
def test_rmsnorm_with_row_gather(dtype, dim, eps):
    from gibbs_b200 import ops
    torch.manual_seed(1)
    x = torch.randn(9, dim) * 3
    g = 1 + 0.1 * torch.randn(dim)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    want = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * g.double()
    out = torch.empty(9, dim, dtype=_dt(dtype), device=DEV)
    ops.rmsnorm(x.to(DEV), g.to(DEV), eps, out)
    _close(out, want, dtype)
    out = torch.empty(3, dim, dtype=_dt(dtype), device=DEV)
    ops.rmsnorm(x.to(DEV), g.to(DEV), eps, out, rows.to(DEV))
    _close(out, want[rows.long()], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    from gibbs_b200 import ops
    torch.manual_seed(2)
    gu, ref = _quant(torch.randn(13, 2 * 200) * 2, dtype)
    out = torch.empty(13, 200, dtype=_dt(dtype), device=DEV)
    ops.swiglu(gu, out)
    g, u = ref[:, :200], ref[:, 200:]
    _close(out, g / (1 + torch.exp(-g)) * u, dtype)


# --------------------------------------------------------------------------- matrix products
SHAPES = [(1, 64, 64), (3, 100, 72), (16, 192, 64), (17, 256, 96), (40, 1000, 200), (64, 2048, 2048),
          (130, 384, 520), (300, 136, 1032), (8, 6144, 2048)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("pair", ["f32xf32", "bf16xbf16", "bf16xf32"])
def test_linear_simt(m, n, k, pair):
    from gibbs_b200 import ops
    torch.manual_seed(m * 7 + n)
    ad, wd = {"f32xf32": ("float32", "float32"), "bf16xbf16": ("bfloat16", "bfloat16"),
              "bf16xf32": ("bfloat16", "float32")}[pair]
    a, ar = _quant(torch.randn(m, k), ad)
    w, wr = _quant(torch.randn(n, k) / math.sqrt(k), wd)
    bias = torch.randn(n)
    want = ar @ wr.T + bias.double()
    out = torch.empty(m, n, dtype=_dt(ad), device=DEV)
    ops.linear_simt(a, w, bias.to(DEV), out)
    _close(out, want, ad)
    res = torch.randn(m, n)
    acc = res.clone().to(DEV)
    ops.linear_simt(a, w, None, acc, accumulate=True)
    _close(acc, res.double() + ar @ wr.T, "float32" if ad == "float32" else "float32", scale=want.abs().max().item())


# the last two split K above 128 rows (few tiles, deep K); the three before them are walked by CTA pairs,
# with ragged edges in both directions
@pytest.mark.parametrize("m,n,k", SHAPES + [(2048, 512, 2048), (1, 65536 // 8, 2048), (257, 130, 8),
                                            (2048, 2048, 256), (1500, 1664, 200), (1281, 2050, 72),
                                            (300, 256, 1024), (520, 392, 4104)])
def test_linear_tensor_cores(m, n, k):
    """bf16 x bf16 on tcgen05: bf16 store, f32 store, f32 accumulate, with and
    without bias, including the split-K sizes."""
    from gibbs_b200 import ops
    torch.manual_seed(m + n + k)
    a, ar = _quant(torch.randn(m, k), "bfloat16")
    w, wr = _quant(torch.randn(n, k) / math.sqrt(k), "bfloat16")
    assert ops.linear_tc_supported(a, w)
    bias = torch.randn(n)
    exact = ar @ wr.T
    scale = exact.abs().max().item()
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.linear_tc(a, w, None, out)
    _close(out, exact, "float32", scale)            # f32 accumulation of exact bf16 products
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(a, w, bias.to(DEV), out)
    _close(out, exact + bias.double(), "bfloat16")
    res = torch.randn(m, n)
    acc = res.clone().to(DEV)
    ops.linear_tc(a, w, bias.to(DEV), acc, accumulate=True)
    _close(acc, res.double() + exact + bias.double(), "float32", scale + 3)
    assert int(ops.device_status(DEV).item()) == 0


def test_linear_tensor_cores_strided_rows():
    """Operands that are column slices of wider rows (their row stride is not their width)."""
    from gibbs_b200 import ops
    torch.manual_seed(5)
    wide, _ = _quant(torch.randn(50, 3 * 128), "bfloat16")
    a = wide[:, 128:256]
    w, wr = _quant(torch.randn(72, 128) / 11, "bfloat16")
    out = torch.empty(50, 72, dtype=torch.float32, device=DEV)
    ops.linear(a, w, None, out)
    _close(out, a.double().cpu() @ wr.T, "float32")


def test_linear_falls_back_when_tma_cannot_address_the_rows():
    from gibbs_b200 import ops
    a, ar = _quant(torch.randn(5, 36), "bfloat16")          # 36 % 8 != 0
    w, wr = _quant(torch.randn(20, 36), "bfloat16")
    assert not ops.linear_tc_supported(a, w)
    out = torch.empty(5, 20, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, None, out)
    _close(out, ar @ wr.T, "bfloat16")


# --------------------------------------------------------------------------- short convolution
def _plain_conv(bcx, taps, bias, state, q_lens):
    """bcx [n, 3h] float64 rows of [B | C | x]; returns (out, new states)."""
    h, k = taps.shape
    outs, new_states, row = [], [], 0
    for r, n in enumerate(q_lens):
        b, c, x = (bcx[row:row + n, i * h:(i + 1) * h] for i in range(3))
        win = torch.cat([state[r], b * x], 0)
        cv = sum(win[j:j + n] * taps[:, j][None, :] for j in range(k))
        if bias is not None:
            cv = cv + bias[None, :]
        outs.append(c * cv)
        new_states.append(win[n:])
        row += n
    return torch.cat(outs, 0), torch.stack(new_states, 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,k,use_bias", [(96, 4, True), (200, 2, False), (64, 7, True)])
def test_short_conv_ragged_batch(dtype, hidden, k, use_bias):
    from gibbs_b200 import ops
    torch.manual_seed(hidden + k)
    q_lens = [1, 5, 2, 1, k - 1, 11]                       # decode tokens, portions shorter than the state, longer ones
    n = sum(q_lens)
    bcx, ref = _quant(torch.randn(n, 3 * hidden), dtype)
    taps = torch.randn(hidden, k)
    bias = torch.randn(hidden) if use_bias else None
    n_slots = 9
    state = torch.randn(n_slots, 2, k - 1, hidden)          # slot axis strided: [slots, 2 (another tenant), k-1, h]
    slot_ids = [7, 0, 3, 8, 2, 5]
    dev_state = state.to(DEV)
    view = dev_state[:, 1]
    q_start = np.cumsum([0] + q_lens[:-1]).astype(np.int32)
    tok_req = np.repeat(np.arange(len(q_lens)), q_lens).astype(np.int32)
    out = torch.empty(n, hidden, dtype=_dt(dtype), device=DEV)
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    ops.short_conv(bcx, taps.to(DEV), None if bias is None else bias.to(DEV), view, t(slot_ids), t(tok_req),
                   t(q_start), t(q_lens), out)
    want, new_state = _plain_conv(ref, taps.double(), None if bias is None else bias.double(),
                                  state[slot_ids, 1].double(), q_lens)
    _close(out, want, dtype)
    got_state = dev_state.cpu()
    assert torch.allclose(got_state[slot_ids, 1].double(), new_state, rtol=1e-6, atol=1e-6)
    untouched = [s for s in range(n_slots) if s not in slot_ids]
    assert torch.equal(got_state[untouched], state[untouched]) and torch.equal(got_state[:, 0], state[:, 0])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,k,use_bias", [(96, 4, True), (200, 2, False), (2048, 3, False)])
def test_short_conv_one_token_per_request(dtype, hidden, k, use_bias):
    """The fused path of decode steps, several steps in a row on the same slots."""
    from gibbs_b200 import ops
    torch.manual_seed(hidden * k)
    n_req, n_slots = 5, 7
    taps = torch.randn(hidden, k)
    bias = torch.randn(hidden) if use_bias else None
    state = torch.randn(n_slots, k - 1, hidden)
    slot_ids = [6, 1, 0, 4, 2]
    dev_state = state.to(DEV)
    ref_state = state[slot_ids].double()
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    for step in range(k + 1):
        bcx, ref = _quant(torch.randn(n_req, 3 * hidden), dtype)
        out = torch.empty(n_req, hidden, dtype=_dt(dtype), device=DEV)
        ops.short_conv(bcx, taps.to(DEV), None if bias is None else bias.to(DEV), dev_state, t(slot_ids),
                       t(list(range(n_req))), t(list(range(n_req))), t([1] * n_req), out, max_q_len=1)
        want, ref_state = _plain_conv(ref, taps.double(), None if bias is None else bias.double(), ref_state,
                                      [1] * n_req)
        _close(out, want, dtype)
        assert torch.allclose(dev_state.cpu()[slot_ids].double(), ref_state, rtol=1e-6, atol=1e-6)
    assert torch.equal(dev_state.cpu()[[3, 5]], state[[3, 5]])


def test_short_conv_refuses_wide_kernels():
    from gibbs_b200 import ops
    from gibbs_b200.ops import KernelError
    z = lambda *s, d=torch.float32: torch.zeros(*s, dtype=d, device=DEV)
    with pytest.raises(KernelError, match="outside 2..16"):
        ops.short_conv(z(1, 24), z(8, 17), None, z(1, 16, 8), z(1, d=torch.int32), z(1, d=torch.int32),
                       z(1, d=torch.int32), torch.ones(1, dtype=torch.int32, device=DEV), z(1, 8))


# --------------------------------------------------------------------------- attention
def _plain_rope(x, pos, inv, rd, adjacent):
    out = x.clone()
    ang = (pos.float()[:, None] * inv.float()[None, :]).double()[:, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    if adjacent:
        a, b = x[..., 0:rd:2], x[..., 1:rd:2]
        out[..., 0:rd:2], out[..., 1:rd:2] = a * c - b * s, a * s + b * c
    else:
        a, b = x[..., :rd // 2], x[..., rd // 2:rd]
        out[..., :rd // 2], out[..., rd // 2:rd] = a * c - b * s, a * s + b * c
    return out


def _layout(lengths_before, q_lens, page_size, n_pages, seed):
    """Random distinct pages for each request; returns metadata arrays."""
    rng = np.random.default_rng(seed)
    perm = rng.permutation(n_pages)
    max_blocks = max(-(-(a + b) // page_size) for a, b in zip(lengths_before, q_lens)) + 1
    bt = np.full((len(q_lens), max_blocks), -1, dtype=np.int32)
    used = 0
    for r, (a, b) in enumerate(zip(lengths_before, q_lens)):
        nb = -(-(a + b) // page_size)
        bt[r, :nb] = perm[used:used + nb]
        used += nb
    assert used <= n_pages
    tok_req = np.repeat(np.arange(len(q_lens)), q_lens).astype(np.int32)
    tok_pos = np.concatenate([np.arange(a, a + b) for a, b in zip(lengths_before, q_lens)]).astype(np.int32)
    return bt, tok_req, tok_pos


CASES = [
    # heads, kv_heads, head_dim, rotary_dim, adjacent, page_size, window, norm
    (4, 2, 16, 16, False, 16, 0, True),
    (3, 1, 32, 32, False, 8, 0, True),
    (6, 3, 48, 32, True, 4, 0, False),
    (8, 2, 64, 64, False, 16, 0, True),
    (5, 5, 80, 80, False, 32, 0, True),
    (2, 1, 128, 64, False, 16, 0, False),
    (4, 2, 16, 16, False, 8, 7, True),
    (8, 8, 8, 8, False, 16, 0, True),
    # bfloat16 portions of 32 tokens and more at head sizes 32, 64, 128 with the whole head rotated take the
    # vector kernel (one block per token); more slots than a block has threads, and no per-head norm
    (32, 8, 64, 64, False, 16, 0, True),
    (40, 40, 128, 128, False, 16, 0, True),
    (2, 1, 128, 128, False, 32, 0, False),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kvh,hd,rd,adjacent,ps,window,norm", CASES)
def test_qk_norm_rope_store_then_attention(dtype, heads, kvh, hd, rd, adjacent, ps, window, norm):
    """A ragged batch against earlier context: requests with 0, some and many
    cached positions, portions and single tokens, pages in random order."""
    from gibbs_b200 import ops
    torch.manual_seed(heads * 100 + hd)
    before = [0, 37, 5, 130, 64]
    q_lens = [9, 1, 20, 1, 3]
    n_pages = 96
    bt, tok_req, tok_pos = _layout(before, q_lens, ps, n_pages, seed=hd)
    n = sum(q_lens)
    width = (heads + 2 * kvh) * hd
    eps = 1e-5
    qkv, ref = _quant(torch.randn(n, width), dtype)
    qg, kg = (1 + 0.2 * torch.randn(hd), 1 + 0.2 * torch.randn(hd)) if norm else (None, None)
    inv = torch.tensor([1.0 / (10000.0 ** (2 * j / rd)) for j in range(rd // 2)], dtype=torch.float32)
    # earlier context: keys/values already in the pages (post-norm, post-rope values, arbitrary)
    k_ctx = [torch.randn(b, kvh, hd) for b in before]
    v_ctx = [torch.randn(b, kvh, hd) for b in before]
    kp = torch.zeros(n_pages, kvh, ps, hd)
    vp = torch.zeros(n_pages, kvh, ps, hd)
    for r, b in enumerate(before):
        for p in range(b):
            kp[bt[r, p // ps], :, p % ps] = k_ctx[r][p]
            vp[bt[r, p // ps], :, p % ps] = v_ctx[r][p]
    kp_d, kp_ref = _quant(kp, dtype)
    vp_d, vp_ref = _quant(vp, dtype)
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    dev = lambda x: None if x is None else x.to(DEV)
    ops.qk_norm_rope_store(qkv, heads, kvh, hd, dev(qg), dev(kg), eps, inv.to(DEV), rd, adjacent, t(tok_req),
                           t(tok_pos), t(bt), kp_d, vp_d, status)
    # plain: norm, rope
    q = ref[:, :heads * hd].reshape(n, heads, hd)
    k = ref[:, heads * hd:(heads + kvh) * hd].reshape(n, kvh, hd)
    v = ref[:, (heads + kvh) * hd:].reshape(n, kvh, hd)
    if norm:
        q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * qg.double()
        k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * kg.double()
    pos = torch.tensor(tok_pos)
    q, k = _plain_rope(q, pos, inv, rd, adjacent), _plain_rope(k, pos, inv, rd, adjacent)
    _close(qkv[:, :heads * hd], q.reshape(n, -1), dtype)
    # the new keys and values landed in their pages; nothing else changed
    kp_want, vp_want = kp_ref.clone(), vp_ref.clone()
    for i in range(n):
        r, p = tok_req[i], tok_pos[i]
        kp_want[bt[r, p // ps], :, p % ps] = k[i]
        vp_want[bt[r, p // ps], :, p % ps] = v[i]
    _close(kp_d, kp_want, dtype)
    _close(vp_d, vp_want, dtype)
    touched = torch.zeros(n_pages, ps, dtype=torch.bool)
    for i in range(n):
        touched[bt[tok_req[i], tok_pos[i] // ps], tok_pos[i] % ps] = True
    assert torch.equal(kp_d.cpu().double()[~touched[:, None, :].expand(-1, kvh, -1)],
                       kp_ref[~touched[:, None, :].expand(-1, kvh, -1)])

    # attention over the pages as the kernel left them (so rounding of stored keys is shared)
    kp_now, vp_now = kp_d.cpu().double(), vp_d.cpu().double()
    q_now = qkv[:, :heads * hd].cpu().double().reshape(n, heads, hd)
    scale = 1.0 / math.sqrt(hd)
    want = torch.zeros(n, heads, hd, dtype=torch.float64)
    for i in range(n):
        r, p = tok_req[i], int(tok_pos[i])
        lo = max(0, p - window + 1) if window else 0
        keys = torch.stack([kp_now[bt[r, j // ps], :, j % ps] for j in range(lo, p + 1)])     # [L, kvh, hd]
        vals = torch.stack([vp_now[bt[r, j // ps], :, j % ps] for j in range(lo, p + 1)])
        for h in range(heads):
            g = h // (heads // kvh)
            s = (keys[:, g] @ q_now[i, h]) * scale
            w = torch.softmax(s, 0)
            want[i, h] = w @ vals[:, g]
    out = torch.empty(n, heads * hd, dtype=_dt(dtype), device=DEV)
    ops.paged_attention(qkv[:, :heads * hd], heads, kvh, hd, kp_d, vp_d, t(bt), t(tok_req), t(tok_pos), scale,
                        window, out, status)
    _close(out, want.reshape(n, -1), dtype)
    assert int(status.item()) == 0


def test_attention_sees_one_far_key_among_hundreds():
    """One key far back is made to dominate: if a page's edge or the lane
    split drops it, the output is visibly wrong."""
    from gibbs_b200 import ops
    heads, kvh, hd, ps = 2, 2, 32, 16
    for length, far in ((700, 0), (700, 15), (700, 16), (513, 511), (1000, 333)):
        torch.manual_seed(far)
        bt = np.arange(-(-length // ps), dtype=np.int32)[None, :]
        kp = torch.randn(64, kvh, ps, hd) * 0.1
        vp = torch.randn(64, kvh, ps, hd)
        q = torch.randn(1, heads * hd) * 0.1
        q[0, :hd] = 4.0                                       # head 0 looks for the far key
        kp[far // ps, 0, far % ps] = 4.0
        vp[far // ps, 0, far % ps] = 100.0
        t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.empty(1, heads * hd, dtype=torch.float32, device=DEV)
        ops.paged_attention(q.to(DEV), heads, kvh, hd, kp.to(DEV), vp.to(DEV), t(bt), t([0]), t([length - 1]),
                            1.0, 0, out, status)
        assert out[0, :hd].min().item() > 99.0, (length, far)
        assert abs(out[0, hd:].mean().item()) < 1.0                 # the other kv head holds no such key


def test_bad_page_id_is_reported_not_dereferenced():
    from gibbs_b200 import ops
    heads, kvh, hd, ps = 2, 1, 16, 4
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kp = torch.zeros(4, kvh, ps, hd, device=DEV)
    out = torch.empty(1, heads * hd, device=DEV)
    ops.paged_attention(torch.zeros(1, heads * hd, device=DEV), heads, kvh, hd, kp, kp.clone(), t([[0, 99, -1]]),
                        t([0]), t([6]), 1.0, 0, out, status)
    assert int(status.item()) == 2
    status.zero_()
    qkv = torch.zeros(1, (heads + 2 * kvh) * hd, device=DEV)
    ops.qk_norm_rope_store(qkv, heads, kvh, hd, None, None, 1e-5, None, 0, False, t([0]), t([5]), t([[0, 4]]),
                           kp, kp.clone(), status)
    assert int(status.item()) == 1


# --------------------------------------------------------------------------- sampling
def test_argmax_first_maximum_and_nan():
    from gibbs_b200 import ops
    x = torch.randn(6, 1000)
    x[0, 17] = x[0, 400] = 50.0                              # tie: the lower id
    x[1, 3] = float("nan")
    x[1, 900] = 60.0
    x[2, :] = float("-inf")
    x[2, 5] = -1e30
    x[3, :] = float("nan")                                   # nothing can win: id 0
    x[4, 999] = 70.0
    x[5, 0] = 70.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.sample(x.to(DEV), out)
    assert out.tolist() == [17, 900, 5, 0, 999, 0]


@pytest.mark.parametrize("vocab", [1000, 65536, 50257])
def test_temperature_sampling_matches_the_plain_rule(vocab):
    """For seeded cases the kernel must pick exactly the candidate the plain
    rule picks with the same uniform number (the reference's test pattern,
    src/runtime/lm.rs:1271-1400)."""
    import plain_lfm2 as plain
    from gibbs_b200 import ops
    from gibbs_b200.sampling import uniform24
    rng = np.random.default_rng(vocab)
    rows = 40
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[3, 10] = logits[3, 20] = logits[3].max() + 1       # a tie at the top
    temp = rng.uniform(0.3, 1.5, rows).astype(np.float32)
    temp[5] = 0.0                                             # greedy row among sampled ones
    top_k = rng.integers(1, 65, rows).astype(np.int32)
    top_p = rng.uniform(0.05, 1.0, rows).astype(np.float32)
    seeds = rng.integers(0, 2 ** 62, rows)
    counters = rng.integers(0, 1000, rows)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(torch.from_numpy(logits).to(DEV), out, torch.from_numpy(temp).to(DEV),
               torch.from_numpy(top_k).to(DEV), torch.from_numpy(top_p).to(DEV),
               torch.from_numpy(seeds.astype(np.int64)).to(DEV), torch.from_numpy(counters.astype(np.int64)).to(DEV))
    got = out.tolist()
    for r in range(rows):
        if temp[r] <= 1e-4:
            assert got[r] == int(np.argmax(logits[r]))
            continue
        ids, probs = plain.nucleus_candidates(logits[r], float(temp[r]), int(top_k[r]), float(top_p[r]))
        u = uniform24(int(seeds[r]), int(counters[r]))
        cum = np.cumsum(probs)
        target = u * cum[-1]
        pick = int(ids[min(int(np.searchsorted(cum, target)), len(ids) - 1)])
        if got[r] != pick:
            # float32 against float64 may disagree only when the draw falls on a boundary
            j = list(ids).index(got[r]) if got[r] in ids else None
            assert j is not None and abs(cum[j - 1 if got[r] != ids[0] and cum[j] > target else j] - target) < 1e-5, r


def test_top_k_selection_with_ties_and_few_finite_values():
    """The candidates are the first k in (logit descending, id ascending) order whatever the row holds:
    thousands of equal values at the threshold (the selection gives way to k passes), equal values
    that still fit, fewer finite values than k, NaNs.  With top_p = 1 and k candidates of equal logit
    the draw u picks candidate floor(u * k), the floor(u * k)-th smallest id."""
    from gibbs_b200 import ops
    from gibbs_b200.sampling import uniform24
    vocab, k = 65536, 37
    rows = []
    a = torch.full((vocab,), -5.0); a[1000:9000] = 2.5                        # 8000 ties above everything else
    b = torch.randn(vocab); b[[7, 77, 777, 7777, 60000]] = 9.0; b[123] = 8.0  # ties that fit; then one more
    c = torch.full((vocab,), float("-inf")); c[[5, 50, 500]] = torch.tensor([1.0, 3.0, 2.0])
    d = torch.randn(vocab); d[::2] = float("nan"); d[40001] = 50.0
    e = torch.zeros(vocab)                                                   # everything ties
    logits = torch.stack([a, b, c, d, e]).to(DEV)
    n = logits.shape[0]
    for seed in range(12):
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        seeds = torch.full((n,), seed, dtype=torch.int64, device=DEV)
        ctr = torch.arange(n, dtype=torch.int64, device=DEV)
        ops.sample(logits, out, torch.full((n,), 1.0, device=DEV), torch.full((n,), k, dtype=torch.int32, device=DEV),
                   torch.full((n,), 1.0, device=DEV), seeds, ctr)
        got = out.tolist()
        u = [uniform24(seed, i) for i in range(n)]
        assert got[0] == 1000 + min(int(u[0] * k), k - 1) or abs(u[0] * k - round(u[0] * k)) < 1e-4
        assert got[4] == min(int(u[4] * k), k - 1) or abs(u[4] * k - round(u[4] * k)) < 1e-4
        assert got[2] in (5, 50, 500) and got[3] % 2 == 1
        # row b: five candidates of logit 9 (weight 1 each), then 8.0 (weight 1/e), then the random rest
        ids_b = [7, 77, 777, 7777, 60000, 123]
        if u[1] < 0.5:
            assert got[1] in ids_b
    # greedy rows through the same kernel (a sampled row beside them): the smallest id of the maxima
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    temp = torch.zeros(n, device=DEV); temp[2] = 1.0
    ops.sample(logits, out, temp, torch.full((n,), k, dtype=torch.int32, device=DEV), torch.full((n,), 1.0, device=DEV),
               torch.zeros(n, dtype=torch.int64, device=DEV), torch.zeros(n, dtype=torch.int64, device=DEV))
    got = out.tolist()
    assert got[0] == 1000 and got[1] == 7 and got[3] == 40001 and got[4] == 0


def test_sampling_distribution():
    from gibbs_b200 import ops
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0] + [-20.0] * 60]).repeat(4000, 1)
    rows = logits.shape[0]
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), out, torch.full((rows,), 1.0, device=DEV),
               torch.full((rows,), 3, dtype=torch.int32, device=DEV), torch.full((rows,), 1.0, device=DEV),
               torch.full((rows,), 1234, dtype=torch.int64, device=DEV), torch.arange(rows, device=DEV))
    counts = np.bincount(out.cpu().numpy(), minlength=4)[:4] / rows
    p = np.exp([2.0, 1.0, 0.0])
    p /= p.sum()
    assert counts[3] == 0 and np.abs(counts[:3] - p).max() < 0.03


# --------------------------------------------------------------------------- tensor-core attention
class _Hints:
    def __init__(self, before, q_lens):
        t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
        self.q_start = t(np.cumsum([0] + list(q_lens[:-1])).tolist())
        self.q_len, self.start_pos = t(q_lens), t(before)
        self.n_requests, self.max_q_len = len(q_lens), max(q_lens)
        self.max_ctx_len = max(a + b for a, b in zip(before, q_lens))


def _plain_paged_attention(q, kp, vp, bt, tok_req, tok_pos, heads, kvh, hd, ps, scale, window):
    n = q.shape[0]
    q = q.reshape(n, heads, hd)
    want = torch.zeros(n, heads, hd, dtype=torch.float64)
    for i in range(n):
        r, p = tok_req[i], int(tok_pos[i])
        lo = max(0, p - window + 1) if window else 0
        idx = torch.arange(lo, p + 1)
        pages = torch.from_numpy(bt[r].astype(np.int64))[idx // ps]
        keys, vals = kp[pages, :, idx % ps], vp[pages, :, idx % ps]          # [L, kvh, hd]
        for h in range(heads):
            g = h // (heads // kvh)
            w = torch.softmax((keys[:, g] @ q[i, h]) * scale, 0)
            want[i, h] = w @ vals[:, g]
    return want.reshape(n, -1)


TC_CASES = [
    # heads, kv_heads, head_dim, page_size, window, lengths before, portion lengths
    (4, 2, 16, 16, 0, [0, 37, 5, 130, 64], [9, 1, 20, 1, 3]),
    (3, 1, 32, 8, 0, [0, 200, 63], [70, 2, 1]),
    (6, 2, 48, 4, 0, [10, 0], [33, 64]),
    (32, 8, 64, 16, 0, [0, 100], [150, 17]),
    (5, 5, 80, 32, 0, [3, 300], [40, 1]),
    (8, 1, 128, 16, 0, [0, 64], [65, 8]),
    (4, 2, 16, 8, 7, [0, 50, 20], [30, 1, 12]),
    (8, 2, 64, 16, 100, [500], [90]),
    # decoding only: one token per request, long contexts, the key range is split among CTAs
    (32, 8, 64, 16, 0, [2047, 5, 700, 64, 63], [1, 1, 1, 1, 1]),
    (4, 1, 32, 16, 0, [1500], [1]),
    (6, 3, 96, 16, 33, [400, 31, 32], [1, 1, 1]),
    (16, 1, 64, 16, 0, [300, 1], [1, 1]),
    (2, 1, 112, 64, 0, [129], [3]),
    # prompt portions at head sizes 64 and 128 (the tcgen05 kernel): every group size, page sizes 8 to 128,
    # windows within a tile and across tiles, decoded tokens beside a portion
    (16, 1, 64, 32, 0, [0, 300], [200, 5]),
    (4, 4, 64, 128, 0, [100], [260]),
    (8, 4, 128, 8, 150, [1000, 0], [40, 300]),
    (32, 8, 64, 16, 0, [2047, 5, 300], [1, 1, 500]),
    (8, 2, 64, 64, 257, [600], [700]),
    (2, 1, 64, 16, 0, [0], [1000]),
    # groups that do not divide the 128 rows of a tile (its last rows stay without a token)
    (24, 8, 64, 16, 0, [0, 1000, 37], [480, 1, 90]),
    (5, 1, 64, 16, 0, [10], [300]),
    (12, 2, 128, 32, 100, [200, 0], [150, 43]),
    (7, 1, 64, 8, 0, [0, 129], [130, 19]),
    (12, 1, 64, 64, 0, [5], [77]),
    # head size 128 in a launch of more than 444 CTAs: key tiles of 64, two CTAs per SM; a window
    (64, 4, 128, 32, 40, [100, 0], [500, 420]),
]


@pytest.mark.parametrize("heads,kvh,hd,ps,window,before,q_lens", TC_CASES)
def test_attention_tensor_cores(heads, kvh, hd, ps, window, before, q_lens):
    from gibbs_b200 import ops
    torch.manual_seed(heads + hd + ps)
    total = sum(a + b for a, b in zip(before, q_lens))
    n_pages = total // ps + len(before) + 8
    bt, tok_req, tok_pos = _layout(before, q_lens, ps, n_pages, seed=hd + ps)
    n = sum(q_lens)
    wide, _ = _quant(torch.randn(n, (heads + 2 * kvh) * hd), "bfloat16")
    q = wide[:, :heads * hd]                                   # a column slice, as the engine passes it
    kp_d, kp = _quant(torch.randn(n_pages, kvh, ps, hd), "bfloat16")
    vp_d, vp = _quant(torch.randn(n_pages, kvh, ps, hd), "bfloat16")
    scale = 1.0 / math.sqrt(hd)
    want = _plain_paged_attention(q.double().cpu(), kp, vp, bt, tok_req, tok_pos, heads, kvh, hd, ps, scale, window)
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((n, heads * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    before_launches = ops.launch_count()
    ops.paged_attention(q, heads, kvh, hd, kp_d, vp_d, t(bt), t(tok_req), t(tok_pos), scale, window, out, status,
                        hints=_Hints(before, q_lens))
    assert ops.attention_tc_supported(q, out, heads, kvh, hd)
    _close(out, want, "bfloat16")
    assert int(status.item()) == 0
    if max(q_lens) == 1 and max(a + 1 for a in before) > 128:
        assert ops.launch_count() - before_launches == 2        # split keys + merge


def test_attention_tensor_cores_far_key_and_tile_edges():
    """A dominant key at the edges of the 64-key tiles and of the splits."""
    from gibbs_b200 import ops
    heads, kvh, hd, ps = 4, 2, 64, 16
    for length, far, q_len in ((700, 0, 1), (700, 63, 1), (700, 64, 1), (1025, 1023, 1), (1000, 333, 1),
                               (300, 255, 40), (300, 256, 40), (129, 128, 129)):
        torch.manual_seed(far)
        nb = -(-length // ps)
        bt = np.arange(nb, dtype=np.int32)[None, :]
        kp = (torch.randn(nb, kvh, ps, hd) * 0.1).to(torch.bfloat16)
        vp = torch.randn(nb, kvh, ps, hd).to(torch.bfloat16)
        q = (torch.randn(q_len, heads * hd) * 0.1).to(torch.bfloat16)
        q[-1, :hd] = 4.0
        kp[far // ps, 0, far % ps] = 4.0
        vp[far // ps, 0, far % ps] = 100.0
        t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.empty(q_len, heads * hd, dtype=torch.bfloat16, device=DEV)
        before = [length - q_len]
        ops.paged_attention(q.to(DEV), heads, kvh, hd, kp.to(DEV), vp.to(DEV), t(bt), t([0] * q_len),
                            t(list(range(length - q_len, length))), 1.0, 0, out, status, hints=_Hints(before, [q_len]))
        assert out[-1, :hd].float().min().item() > 99.0, (length, far, q_len)
        assert abs(out[-1, 2 * hd:].float().mean().item()) < 1.0


@pytest.mark.parametrize("m,f,k", [(1, 64, 64), (8, 192, 96), (8, 8192, 2048), (64, 256, 2048), (300, 448, 136),
                                   (2, 128, 4096), (2048, 1280, 128), (1300, 1024, 200)])
@pytest.mark.parametrize("use_bias", [False, True])
def test_linear_tensor_cores_swiglu_epilogue(m, f, k, use_bias):
    """gate and up as one product whose epilogue applies (g * sigmoid(g)) * u,
    directly and through the split-K path."""
    from gibbs_b200 import ops
    from gibbs_b200.parts.linear import interleave_gate_up
    torch.manual_seed(m + f + k)
    a, ar = _quant(torch.randn(m, k), "bfloat16")
    wg, wgr = _quant(torch.randn(f, k) / math.sqrt(k) * 2, "bfloat16")
    wu, wur = _quant(torch.randn(f, k) / math.sqrt(k) * 2, "bfloat16")
    bg, bu = torch.randn(f), torch.randn(f)
    w = interleave_gate_up(wg, wu)
    bias = interleave_gate_up(bg, bu).to(DEV) if use_bias else None
    g = ar @ wgr.T + (bg.double() if use_bias else 0)
    u = ar @ wur.T + (bu.double() if use_bias else 0)
    want = g / (1 + torch.exp(-g)) * u
    out = torch.full((m, f), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(a, w, bias, out, swiglu=True)
    _close(out, want, "bfloat16")
    assert int(ops.device_status(DEV).item()) == 0


def test_deferred_split_k_and_norm_that_adds_the_partial_sums():
    """A product into the residual stream that splits K leaves partial sums;
    the norm adds them in split order, writes the stream back and normalises."""
    from gibbs_b200 import ops
    torch.manual_seed(11)
    m, n, k, eps = 8, 256, 2048, 1e-5
    a, ar = _quant(torch.randn(m, k), "bfloat16")
    w, wr = _quant(torch.randn(n, k) / math.sqrt(k), "bfloat16")
    bias, gain = torch.randn(n), 1 + 0.1 * torch.randn(n)
    x0 = torch.randn(m, n)
    x = x0.clone().to(DEV)
    ws = ops.linear_tc(a, w, bias.to(DEV), x, accumulate=True, defer=True)
    assert ws is not x and ws.shape[1:] == (m, n) and ws.shape[0] > 1
    assert torch.equal(x.cpu(), x0)                                  # nothing was added yet
    want_x = x0.double() + ar @ wr.T + bias.double()
    want_h = want_x / torch.sqrt((want_x ** 2).mean(-1, keepdim=True) + eps) * gain.double()
    # gathered rows: the stream itself stays as it was
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(3, n, dtype=torch.float32, device=DEV)
    ops.rmsnorm(x, gain.to(DEV), eps, out, rows, pending=(ws, bias.to(DEV)))
    _close(out, want_h[[5, 0, 5]], "float32")
    assert torch.equal(x.cpu(), x0)
    # all rows: normalised output and the stream updated
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x, gain.to(DEV), eps, out, None, pending=(ws, bias.to(DEV)))
    _close(out, want_h, "bfloat16")
    _close(x, want_x, "float32")
    # and the plain way of adding them
    x2 = x0.clone().to(DEV)
    ops.add_pending(x2, ws, bias.to(DEV))
    assert torch.equal(x2, x)


def test_split_k_above_128_rows_is_left_to_the_norm_too():
    """A prompt portion against a narrow, deep weight splits K as well (few tiles would leave most
    SMs idle); its partial tiles reach the norm like the decode sizes' do."""
    from gibbs_b200 import ops
    torch.manual_seed(12)
    m, n, k, eps = 300, 256, 4096, 1e-5
    a, ar = _quant(torch.randn(m, k), "bfloat16")
    w, wr = _quant(torch.randn(n, k) / math.sqrt(k), "bfloat16")
    gain = 1 + 0.1 * torch.randn(n)
    x0 = torch.randn(m, n)
    x = x0.clone().to(DEV)
    ws = ops.linear_tc(a, w, None, x, accumulate=True, defer=True)
    assert ws is not x and ws.shape == (8, m, n)
    want_x = x0.double() + ar @ wr.T
    want_h = want_x / torch.sqrt((want_x ** 2).mean(-1, keepdim=True) + eps) * gain.double()
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x, gain.to(DEV), eps, out, None, pending=(ws, None))
    _close(out, want_h, "bfloat16")
    _close(x, want_x, "float32", scale=want_x.abs().max().item())


@pytest.mark.parametrize("before,q_len,window,far", [
    (1499, 1, 0, 0), (1499, 1, 0, 15), (1499, 1, 0, 16), (1499, 1, 0, 767), (1499, 1, 0, 1499),   # decode, key splits
    (1499, 1, 300, 1200), (1499, 1, 300, 1199),                    # the window's first key, and the one before it
    (1000, 200, 0, 3), (1000, 200, 0, 1127), (1000, 200, 0, 1128),  # a portion: tile and page edges
    (1000, 200, 150, 1000), (0, 333, 64, 130),                      # a window that some rows of the portion have left
])
def test_tensor_core_attention_sees_one_far_key_and_the_windows_edge(before, q_len, window, far):
    """bfloat16 kernels (key splits when decoding, tcgen05 for the portion): one key is made to
    dominate head 0 of every query row.  A row sees it exactly when the key is not after the row
    and inside its window; a key lost at a page's, a tile's or a split's edge, or let in from
    outside the window, shows as 100 against about 0."""
    from gibbs_b200 import ops
    heads, kvh, hd, ps = 8, 2, 64, 16
    torch.manual_seed(far + window)
    total = before + q_len
    n_pages = total // ps + 6
    bt, tok_req, tok_pos = _layout([before], [q_len], ps, n_pages, seed=far)
    kp = torch.randn(n_pages, kvh, ps, hd) * 0.05
    vp = torch.randn(n_pages, kvh, ps, hd) * 0.5
    kp[bt[0, far // ps], 0, far % ps] = 4.0
    vp[bt[0, far // ps], 0, far % ps] = 100.0
    q = torch.randn(q_len, heads * hd) * 0.05
    q[:, :hd] = 4.0                                            # head 0 (kv head 0) of every row looks for the key
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((q_len, heads * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q.to(DEV).to(torch.bfloat16), heads, kvh, hd, kp.to(DEV).to(torch.bfloat16),
                        vp.to(DEV).to(torch.bfloat16), t(bt), t(tok_req), t(tok_pos), 1.0 / 8, window, out, status,
                        hints=_Hints([before], [q_len]))
    assert int(status.item()) == 0
    got = out.float().cpu()
    for i in range(q_len):
        pos = before + i
        visible = far <= pos and (window == 0 or far + window > pos)
        head0 = got[i, :hd]
        if visible:
            assert head0.min().item() > 99.0, (i, pos)
        else:
            assert head0.abs().max().item() < 3.0, (i, pos)
        assert got[i, hd:].abs().max().item() < 3.0              # no other head holds such a key


# --------------------------------------------------------------------------- consumers of split-K partial tiles
def _split_partials(full: torch.Tensor, splits: int, seed: int):
    """Random 32-bit partial tiles [splits, m, n] whose sum in split order is what a reduction
    kernel would compute; returns (tiles on the device, their bfloat16-rounded sum)."""
    g = torch.Generator().manual_seed(seed)
    parts = torch.randn(splits, *full.shape, generator=g) * 0.3
    parts[0] = full - parts[1:].sum(0)
    acc = torch.zeros_like(full)
    for s in range(splits):                     # the order the kernels add in
        acc = acc + parts[s]
    return parts.to(DEV), acc


@pytest.mark.gpu
@pytest.mark.parametrize("hidden,k,splits,use_bias", [(96, 4, 3, True), (200, 2, 1, False), (2048, 3, 9, False)])
def test_short_conv_from_partial_tiles_equals_the_two_kernel_way(hidden, k, splits, use_bias):
    from gibbs_b200 import ops
    torch.manual_seed(hidden + splits)
    n_req, n_slots = 5, 7
    taps, bias = torch.randn(hidden, k), (torch.randn(hidden) if use_bias else None)
    in_bias = torch.randn(3 * hidden) if use_bias else None
    state = torch.randn(n_slots, k - 1, hidden)
    slot_ids = [6, 1, 0, 4, 2]
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    dev = lambda x: None if x is None else x.to(DEV)
    st_a, st_b = state.to(DEV), state.to(DEV)
    for step in range(3):
        ws, total = _split_partials(torch.randn(n_req, 3 * hidden), splits, seed=step)
        if in_bias is not None:
            total = total + in_bias
        bcx = total.to(torch.bfloat16).to(DEV)                        # what the reduction kernel would have written
        want = torch.empty(n_req, hidden, dtype=torch.bfloat16, device=DEV)
        ops.short_conv(bcx, dev(taps), dev(bias), st_a, t(slot_ids), t(list(range(n_req))), t(list(range(n_req))),
                       t([1] * n_req), want, max_q_len=1)
        got = torch.empty_like(want)
        ops.short_conv_partials(ops.Partials(ws, dev(in_bias), torch.bfloat16), dev(taps), dev(bias), st_b,
                                t(slot_ids), t(list(range(n_req))), got)
        assert torch.equal(got, want)
        assert torch.equal(st_a, st_b)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kvh,hd,rd,adjacent,norm,splits,write_kv",
                         [(4, 2, 16, 16, False, True, 2, True), (3, 1, 32, 16, True, False, 5, True),
                          (32, 8, 64, 64, False, True, 6, True), (2, 2, 128, 128, False, True, 1, False),
                          (5, 5, 80, 40, False, True, 3, True)])
def test_qk_norm_rope_store_from_partial_tiles_equals_the_two_kernel_way(heads, kvh, hd, rd, adjacent, norm, splits,
                                                                         write_kv):
    from gibbs_b200 import ops
    torch.manual_seed(heads * 10 + hd)
    before, q_lens, ps, n_pages = [0, 37, 5], [4, 1, 1], 8, 40
    bt, tok_req, tok_pos = _layout(before, q_lens, ps, n_pages, seed=hd)
    n = sum(q_lens)
    cols = (heads + (2 * kvh if write_kv else 0)) * hd
    bias = torch.randn(cols)
    ws, total = _split_partials(torch.randn(n, cols), splits, seed=3)
    qkv = (total + bias).to(torch.bfloat16).to(DEV)
    qg, kg = ((1 + 0.2 * torch.randn(hd)).to(DEV), (1 + 0.2 * torch.randn(hd)).to(DEV)) if norm else (None, None)
    inv = torch.tensor([1.0 / (10000.0 ** (2 * j / rd)) for j in range(rd // 2)], dtype=torch.float32, device=DEV)
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pages = lambda: (torch.zeros(n_pages, kvh, ps, hd, dtype=torch.bfloat16, device=DEV) if write_kv else None)
    kp_a, vp_a, kp_b, vp_b = pages(), pages(), pages(), pages()
    ops.qk_norm_rope_store(qkv, heads, kvh, hd, qg, kg, 1e-5, inv, rd, adjacent, t(tok_req), t(tok_pos), t(bt),
                           kp_a, vp_a, status)
    q = torch.empty(n, heads * hd, dtype=torch.bfloat16, device=DEV)
    ops.qk_norm_rope_store_partials(ops.Partials(ws, bias.to(DEV), torch.bfloat16), q, heads, kvh, hd, qg, kg, 1e-5,
                                    inv, rd, adjacent, t(tok_req), t(tok_pos), t(bt), kp_b, vp_b, status)
    assert torch.equal(q, qkv[:, :heads * hd])
    if write_kv:
        assert torch.equal(kp_a, kp_b) and torch.equal(vp_a, vp_b)
        assert kp_a.abs().sum() > 0
    assert int(status.item()) == 0


@pytest.mark.gpu
def test_linear_partials_returns_tiles_only_when_k_is_split():
    from gibbs_b200 import ops
    torch.manual_seed(5)
    a, ar = _quant(torch.randn(8, 2048), "bfloat16")
    w, wr = _quant(torch.randn(384, 2048) / 45.0, "bfloat16")        # 3 tiles of weight rows: K is split
    bias = torch.randn(384, device=DEV)
    p = ops.linear_tc_partials(a, w, bias)
    assert isinstance(p, ops.Partials) and p.ws.shape[0] > 1 and p.shape == (8, 384)
    _close(p.ws.sum(0) + bias, ar @ wr.T + bias.cpu().double(), "float32")
    w2, w2r = _quant(torch.randn(128 * 100, 64) / 8.0, "bfloat16")   # many tiles: no split, finished product
    a2, a2r = _quant(torch.randn(8, 64), "bfloat16")
    out = ops.linear_tc_partials(a2, w2, None)
    assert isinstance(out, torch.Tensor) and out.dtype == torch.bfloat16
    _close(out, a2r @ w2r.T, "bfloat16")


# --------------------------------------------------------------------------- decode products (cluster split-K, fused norm)
DECODE_SHAPES = [(1, 64, 64), (8, 2048, 2048), (8, 6144, 2048), (8, 3072, 2048), (8, 2048, 8192), (3, 100, 72),
                 (16, 192, 64), (17, 256, 96), (40, 1000, 200), (64, 2048, 2048), (64, 1536, 6912), (33, 136, 1032),
                 (1, 65536 // 8, 2048), (5, 4608, 1536)]


@pytest.mark.parametrize("m,n,k", DECODE_SHAPES)
def test_linear_decode_against_float64(m, n, k):
    """Every store of the decode product, with K split inside a cluster where the weight has few
    tiles (1 to 8 ranks, slices of rows that do not divide 128), ragged edges in n and k."""
    from gibbs_b200 import ops
    torch.manual_seed(m + n + k)
    a, ar = _quant(torch.randn(m, k), "bfloat16")
    w, wr = _quant(torch.randn(n, k) / math.sqrt(k), "bfloat16")
    assert ops.linear_decode_supported(m, w)
    bias = torch.randn(n)
    exact = ar @ wr.T
    scale = exact.abs().max().item()
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.linear_decode(a, w, None, out)
    _close(out, exact, "float32", scale)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_decode(a, w, bias.to(DEV), out)
    _close(out, exact + bias.double(), "bfloat16")
    # into the residual stream, with the partial sums of squares of the new rows
    x0 = torch.randn(m, n)
    x = x0.clone().to(DEV)
    ssq = ops.linear_decode(a, w, bias.to(DEV), x, accumulate=True, want_ssq=True)
    want_x = x0.double() + exact + bias.double()
    _close(x, want_x, "float32", scale=want_x.abs().max().item())
    assert ssq.shape[1] == m
    got_ss = ssq.double().sum(0).cpu()
    want_ss = (want_x ** 2).sum(-1)
    assert ((got_ss - want_ss).abs() / want_ss).max().item() < 1e-5
    assert int(ops.device_status(DEV).item()) == 0


@pytest.mark.parametrize("m,n,k,gather", [(1, 256, 64, False), (8, 6144, 2048, False), (8, 3072, 2048, False),
                                          (8, 8192, 2048, True), (3, 200, 72, True), (16, 1000, 200, False),
                                          (12, 4608, 1536, False), (16, 384, 2048, True), (8, 16384, 2048, False),
                                          (5, 256, 4096, False)])
@pytest.mark.parametrize("with_ssq", [False, True])
def test_linear_decode_with_the_norm_inside(m, n, k, gather, with_ssq):
    """x_mode 1: the product reads the 32-bit stream through an RMSNorm of its own (scale from the
    row or from partial sums of squares), with and without a row gather."""
    from gibbs_b200 import ops
    torch.manual_seed(m * 3 + n + k)
    eps = 1e-5
    n_src = m + 3 if gather else m
    x = torch.randn(n_src, k) * 2
    gain = 1 + 0.1 * torch.randn(k)
    w, wr = _quant(torch.randn(n, k) / math.sqrt(k), "bfloat16")
    rows = torch.randperm(n_src)[:m].to(torch.int32) if gather else None
    src = x[rows.long()] if gather else x
    h = src.double() / torch.sqrt((src.double() ** 2).mean(-1, keepdim=True) + eps) * gain.double()
    h_bf = h.to(torch.bfloat16).double()                       # what the kernel's operand is rounded to
    want = h_bf @ wr.T
    ssq = None
    if with_ssq:
        # partial sums over three uneven column ranges, as a product before would have left them
        cuts = [0, k // 3, k // 2, k]
        ssq = torch.stack([(x[:, a:b] ** 2).sum(-1) for a, b in zip(cuts[:-1], cuts[1:])]).contiguous().to(DEV)
    a = ops.NormedRows(x.to(DEV), gain.to(DEV), eps, None if rows is None else rows.to(DEV), ssq)
    assert ops.linear_decode_normed_ok(m, n, k) and not ops.linear_decode_normed_ok(17, n, k)
    assert not ops.linear_decode_normed_ok(m, 65536, k)          # more tiles than one wave of CTAs: the norm runs by itself
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.linear_decode(a, w, None, out)
    # the operand's rounding to bfloat16 may fall the other way for values at a rounding edge
    _close(out, want, "float32", scale=want.abs().max().item() * 200)
    _close(out, h @ wr.T, "bfloat16")
    assert int(ops.device_status(DEV).item()) == 0


@pytest.mark.parametrize("m,f,k", [(1, 64, 64), (8, 8192, 2048), (8, 192, 96), (64, 256, 2048), (2, 128, 4096),
                                   (33, 448, 136)])
@pytest.mark.parametrize("normed", [False, True])
def test_linear_decode_swiglu(m, f, k, normed):
    from gibbs_b200 import ops
    from gibbs_b200.parts.linear import interleave_gate_up
    if normed and m > 16:
        pytest.skip("the norm runs inside the product for up to 16 rows")
    torch.manual_seed(m + f + k)
    wg, wgr = _quant(torch.randn(f, k) / math.sqrt(k) * 2, "bfloat16")
    wu, wur = _quant(torch.randn(f, k) / math.sqrt(k) * 2, "bfloat16")
    bg, bu = torch.randn(f), torch.randn(f)
    w = interleave_gate_up(wg, wu)
    bias = interleave_gate_up(bg, bu).to(DEV)
    if normed:
        x = torch.randn(m, k) * 3
        gain = 1 + 0.1 * torch.randn(k)
        ar = (x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6) * gain.double())
        a = ops.NormedRows(x.to(DEV), gain.to(DEV), 1e-6)
    else:
        a, ar = _quant(torch.randn(m, k), "bfloat16")
    g = ar @ wgr.T + bg.double()
    u = ar @ wur.T + bu.double()
    want = g / (1 + torch.exp(-g)) * u
    out = torch.full((m, f), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_decode(a, w, bias, out, swiglu=True)
    _close(out, want, "bfloat16")
    assert int(ops.device_status(DEV).item()) == 0


# --------------------------------------------------------------------------- a bounded wait that runs out
BOUNDED_WAIT_SOURCE = r'''
#include "sm100.cuh"

// One thread waits, with a limit of a millisecond, for a phase of an mbarrier that nobody ever arrives
// at (no copy is in flight, no tensor memory is held); the wait gives up, the kernel records a code
// in the status word as the tensor-core kernels do, and returns.
__global__ void bounded_wait_kernel(int* status, int* polls_done) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    sm100::fence_barrier_init();
    const bool ok = sm100::mbar_wait<1000>(&bar, 0);
    *polls_done = ok ? 0 : 1;
    if (!ok) atomicExch(status, 16 + 7);
  }
}

extern "C" __attribute__((visibility("default")))
int bounded_wait_probe(int* status, int* polls_done, cudaStream_t stream) {
  bounded_wait_kernel<<<1, 32, 0, stream>>>(status, polls_done);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
'''


def test_a_bounded_wait_that_runs_out_sets_the_status_word_and_the_engine_reports_it(tmp_path):
    """Every mbarrier wait of the tensor-core kernels is bounded (csrc/sm100.cuh); here one runs out
    on purpose, in a kernel of the test's own that holds nothing: the kernel returns, the context
    stays usable, the status word carries the code and the engine turns it into an error."""
    import ctypes
    import subprocess
    from gibbs_b200 import Engine, Lfm2Config, ops, random_model
    from gibbs_b200.csrc import build
    from gibbs_b200.engine.step import StepEntry, StepError
    from helpers import TINY_A
    src, so = tmp_path / "bounded_wait.cu", tmp_path / "libbounded_wait.so"
    src.write_text(BOUNDED_WAIT_SOURCE)
    subprocess.run([build.find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-shared", "-Xcompiler",
                    "-fPIC", "-I", str(build.HERE), str(src), "-o", str(so)], check=True)
    lib = ctypes.CDLL(str(so))
    eng = Engine(random_model(Lfm2Config.from_dict(TINY_A), 0, dtype="float32"), n_pages=4, page_size=16,
                 max_requests=1, max_step_tokens=16)
    status = ops.device_status(DEV)
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert int(status.item()) == 0
    assert lib.bounded_wait_probe(ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(gave_up.data_ptr()),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()                                   # the kernel returned by itself
    assert int(gave_up.item()) == 1 and int(status.item()) == 23
    with pytest.raises(StepError, match="bounded wait.*ran out.*23"):
        eng.check_status()
    assert int(status.item()) == 0                             # reported once, then cleared
    # the context is as usable as before
    eng.open("r")
    assert eng.step([StepEntry("r", [1, 2, 3], [2])]).shape == (1, TINY_A["vocab_size"])
    eng.check_status()
    eng.close("r")


@pytest.mark.parametrize("pair", ["f32xf32", "bf16xf32"])
def test_linear_simt_gives_the_same_bits_however_the_rows_are_cut(pair):
    """The 32-bit product has three kernels (128 x 128 tiles for prompts, 16-column tiles for a few
    rows, a general one): every output is one accumulator walking k upwards in each of them, so a row
    has the same bits whether it comes alone, among 16, among 64 or among 200."""
    from gibbs_b200 import ops
    torch.manual_seed(3)
    ad = "float32" if pair == "f32xf32" else "bfloat16"
    m, n, k = 200, 392, 2048
    a, ar = _quant(torch.randn(m, k), ad)
    w, wr = _quant(torch.randn(n, k) / math.sqrt(k), "float32")
    bias = torch.randn(n).to(DEV)
    whole = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.linear_simt(a, w, bias, whole)
    _close(whole, ar @ wr.T + bias.double().cpu(), "float32")
    for lo, hi in ((0, 1), (1, 17), (17, 81), (81, 200), (5, 13)):
        part = torch.empty(hi - lo, n, dtype=torch.float32, device=DEV)
        ops.linear_simt(a[lo:hi], w, bias, part)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)


@pytest.mark.parametrize("vocab,k", [(1000, 5), (65536, 20), (50257, 1), (7, 32)])
def test_logprob_info_matches_the_plain_rule(vocab, k):
    """Probability of the chosen token, entropy and the k most probable tokens of every row,
    against the reference's rule restated in float64 (src/scheduler/mod.rs:272-315); ties are
    ordered by id, NaNs never count, rows with fewer than k numbers are padded with -1."""
    from gibbs_b200 import ops
    torch.manual_seed(vocab + k)
    rows = 5
    logits = torch.randn(rows, vocab) * 3
    logits[1, : min(vocab, 4)] = 9.0                       # a tie at the top: lowest ids first
    logits[2, ::2] = float("nan")
    if vocab > 100:
        logits[3, 50:] = float("nan")                      # fewer numbers than some k
    chosen = torch.tensor([0, 1, 1, 3, vocab - 1], dtype=torch.int32)
    prob, ent, ids, probs = ops.logprob_info(logits.to(DEV), chosen.to(DEV), k)
    for r in range(rows):
        row = logits[r].double()
        ok = ~torch.isnan(row)
        lse = torch.logsumexp(row[ok], 0)
        p = torch.where(ok, torch.exp(row - lse), torch.zeros_like(row))
        want_ent = float(-(p[ok] * (row[ok] - lse))[p[ok] > 1e-12].sum())
        assert abs(ent[r].item() - want_ent) < 1e-3 * max(1.0, abs(want_ent))
        assert abs(prob[r].item() - min(float(p[chosen[r]]), 1.0)) < 1e-5
        order = sorted((i for i in range(vocab) if ok[i]), key=lambda i: (-float(row[i]), i))[:k]
        got = [int(i) for i in ids[r].tolist()]
        assert got[:len(order)] == order and all(i == -1 for i in got[len(order):])
        for j, i in enumerate(order):
            assert abs(probs[r, j].item() - float(p[i])) < 1e-5


# --------------------------------------------------------------------------- kernels of a decode step: one trip to L2
@pytest.mark.gpu
@pytest.mark.parametrize("n,dim,splits,use_bias,gather", [
    (8, 2048, 9, False, False), (1, 2048, 16, True, False), (64, 1536, 8, False, False), (5, 1000, 3, True, True),
    (3, 4096, 9, False, False), (2, 8192, 4, False, False), (2, 8192, 9, True, False), (7, 72, 2, False, True),
    (4, 66, 5, True, False)])
def test_rmsnorm_adds_the_partial_sums_of_many_splits_in_split_order(n, dim, splits, use_bias, gather):
    """The norm that follows a split-K product: every variant (partial sums through shared memory,
    in registers when they do not fit there, element by element for rows of no 16-byte pieces)
    against the sum formed in split order in 32-bit and a float64 norm."""
    from gibbs_b200 import ops
    torch.manual_seed(n + dim + splits)
    eps = 1e-5
    x0 = torch.randn(n, dim)
    ws = torch.randn(splits, n, dim) * 0.3
    bias = torch.randn(dim) if use_bias else None
    gain = 1 + 0.1 * torch.randn(dim)
    total = x0.clone()
    for s in range(splits):
        total = total + ws[s]                              # float32, split order: the kernel's own order
    if use_bias:
        total = total + bias
    t64 = total.double()
    want_h = t64 / torch.sqrt((t64 ** 2).mean(-1, keepdim=True) + eps) * gain.double()
    x = x0.clone().to(DEV)
    pend = (ws.to(DEV), bias.to(DEV) if use_bias else None)
    if gather:
        rows = torch.tensor([n - 1, 0], dtype=torch.int32, device=DEV)
        out = torch.empty(2, dim, dtype=torch.float32, device=DEV)
        ops.rmsnorm(x, gain.to(DEV), eps, out, rows, pending=pend)
        _close(out, want_h[[n - 1, 0]], "float32")
        assert torch.equal(x.cpu(), x0)
    else:
        out = torch.empty(n, dim, dtype=torch.float32, device=DEV)
        ops.rmsnorm(x, gain.to(DEV), eps, out, None, pending=pend)
        _close(out, want_h, "float32")
        assert torch.equal(x.cpu(), total)                 # the stream carries the sum, bit for bit


@pytest.mark.gpu
def test_qk_norm_rope_store_from_partial_tiles_that_are_not_16_byte_aligned():
    """Partial tiles that start 4 bytes off a 16-byte boundary take the kernel's plain loads instead
    of its 16-byte copies; same bits either way."""
    from gibbs_b200 import ops
    torch.manual_seed(77)
    heads, kvh, hd, rd, splits = 6, 2, 64, 64, 6
    before, q_lens, ps, n_pages = [9, 37, 5], [1, 1, 1], 8, 40
    bt, tok_req, tok_pos = _layout(before, q_lens, ps, n_pages, seed=hd)
    n = sum(q_lens)
    cols = (heads + 2 * kvh) * hd
    ws, total = _split_partials(torch.randn(n, cols), splits, seed=3)
    buf = torch.empty(ws.numel() + 1, dtype=torch.float32, device=DEV)
    off = buf[1:].view(ws.shape)
    off.copy_(ws)
    assert off.data_ptr() % 16 == 4 and ws.data_ptr() % 16 == 0
    qg, kg = (1 + 0.2 * torch.randn(hd)).to(DEV), (1 + 0.2 * torch.randn(hd)).to(DEV)
    inv = torch.tensor([1.0 / (10000.0 ** (2 * j / rd)) for j in range(rd // 2)], dtype=torch.float32, device=DEV)
    t = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pages = lambda: torch.zeros(n_pages, kvh, ps, hd, dtype=torch.bfloat16, device=DEV)
    kp_a, vp_a, kp_b, vp_b = pages(), pages(), pages(), pages()
    qa = torch.empty(n, heads * hd, dtype=torch.bfloat16, device=DEV)
    qb = torch.empty_like(qa)
    for w, q, kp, vp in ((ws, qa, kp_a, vp_a), (off, qb, kp_b, vp_b)):
        ops.qk_norm_rope_store_partials(ops.Partials(w, None, torch.bfloat16), q, heads, kvh, hd, qg, kg, 1e-5, inv, rd,
                                        False, t(tok_req), t(tok_pos), t(bt), kp, vp, status)
    assert torch.equal(qa, qb) and torch.equal(kp_a, kp_b) and torch.equal(vp_a, vp_b)
    assert qa.float().abs().sum() > 0 and kp_a.float().abs().sum() > 0 and int(status.item()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [65536, 50001, 8192, 8200])
def test_argmax_over_a_cluster_of_blocks(vocab):
    """Rows of 8,192 and more are scanned by eight blocks each: ties across their slices go to the
    lower id, NaN never wins, a maximum at a slice's edge is found."""
    from gibbs_b200 import ops
    torch.manual_seed(vocab)
    per = (((vocab + 7) // 8) + 3) // 4 * 4
    x = torch.randn(9, vocab)
    x[0, per - 1] = x[0, per] = 50.0                         # tie across two slices
    x[1, 3] = float("nan")
    x[1, vocab - 1] = 60.0                                   # the last element
    x[2, :] = float("-inf")
    x[2, 5 * per + 1] = -1e30
    x[3, :] = float("nan")                                   # nothing can win: id 0
    x[4, 7 * per] = 70.0                                     # first element of the last slice
    x[5, 0] = 70.0
    x[6, 3 * per - 1] = 80.0                                 # last element of a slice
    x[7, 6 * per + 2] = x[7, 2 * per + 2] = 90.0             # tie far apart
    out = torch.empty(9, dtype=torch.int32, device=DEV)
    ops.sample(x.to(DEV), out)
    want = [per - 1, vocab - 1, 5 * per + 1, 0, 7 * per, 0, 3 * per - 1, 2 * per + 2, int(torch.argmax(x[8]))]
    assert out.tolist() == want


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [1000, 65536])
def test_repetition_penalty_matches_the_plain_rule(vocab):
    """Greedy and sampling rows, tokens that occur once, several times and not at all, positive
    and negative logits, rows with fewer than 64 recent tokens, a row whose penalty is off and a
    token id outside the vocabulary (ignored)."""
    import plain_lfm2 as plain
    from gibbs_b200 import ops
    rng = np.random.default_rng(vocab)
    rows = 6
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    recent = [list(rng.integers(0, vocab, 64)), [5, 5, 5, 7, 5], [], list(rng.integers(0, 20, 64)), [1, 2, 3],
              [9, vocab + 3, 9]]
    logits[1, 5], logits[1, 7] = 4.0, -2.0
    penalty = np.array([1.3, 2.0, 1.5, 1.1, 1.0, 1.7], dtype=np.float32)
    temperature = np.array([0.0, 0.8, 0.0, 1.2, 0.7, 0.0], dtype=np.float32)
    ids = np.full((rows, 64), -1, dtype=np.int32)
    for r, toks in enumerate(recent):
        ids[r, :len(toks)] = toks
    got = ops.repetition_penalty(torch.from_numpy(logits).to(DEV), torch.from_numpy(ids).to(DEV),
                                 torch.from_numpy(penalty).to(DEV), torch.from_numpy(temperature).to(DEV)).cpu().numpy()
    for r in range(rows):
        want = plain.penalized(logits[r], recent[r], float(penalty[r]), temperature[r] <= 1e-4)
        assert np.array_equal(got[r], want), r
    assert not np.array_equal(got[0], logits[0]) and np.array_equal(got[4], logits[4]) and np.array_equal(got[2], logits[2])
    # all rows greedy when no temperatures are given
    got = ops.repetition_penalty(torch.from_numpy(logits).to(DEV), torch.from_numpy(ids).to(DEV),
                                 torch.from_numpy(penalty).to(DEV)).cpu().numpy()
    assert np.array_equal(got[1], plain.penalized(logits[1], recent[1], 2.0, True))
