"""Grouped-query causal attention over the paged cache.

q, k, v projections (one fused product), optional per-head RMSNorm of q and k
before the rotary encoding, keys and values written into the request's pages,
softmax((q.K) * scale) V over the visible keys, output projection added into
the residual stream (MisterTK/gibbs arch/lib/transformer.json5:46-87;
src/graph/cpu.rs:826-951).  ``window`` keeps the last ``window`` keys visible
only; ``shares_kv`` makes the layer read a cache another entry writes: it
then has no k/v projections of its own (transformer.json5:39-41, write: false).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, PagedKV, TensorDecl, VECTOR, part_class, register_part
from .linear import Linear


class GQAAttention(Mixer):
    fuses_norm = True          # its input goes straight into a product (parts.linear.Linear)

    @classmethod
    def declare(cls, params):
        h, hd = params["hidden"], params["head_dim"]
        a, kvd = params["heads"] * hd, params["kv_heads"] * hd
        shares = params.get("shares_kv", False)
        d = {"q_proj.weight": TensorDecl.of(a, h), "out_proj.weight": TensorDecl.of(h, a)}
        if not shares:
            d["k_proj.weight"] = TensorDecl.of(kvd, h)
            d["v_proj.weight"] = TensorDecl.of(kvd, h)
        if params.get("qk_norm"):
            d["q_norm.weight"] = TensorDecl.of(hd, role=VECTOR)
            if not shares:
                d["k_norm.weight"] = TensorDecl.of(hd, role=VECTOR)
        if params.get("bias"):
            d["q_proj.bias"] = TensorDecl.of(a, role=VECTOR)
            d["out_proj.bias"] = TensorDecl.of(h, role=VECTOR)
            if not shares:
                d["k_proj.bias"] = TensorDecl.of(kvd, role=VECTOR)
                d["v_proj.bias"] = TensorDecl.of(kvd, role=VECTOR)
        return d

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hidden, self.heads = int(params["hidden"]), int(params["heads"])
        self.kv_heads, self.head_dim = int(params["kv_heads"]), int(params["head_dim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        self.scale = float(params["scale"])
        self.window = params.get("window")
        self.shares_kv = bool(params.get("shares_kv", False))
        self.eps = float(params.get("qk_norm_eps", 0.0))
        # scores pass through cap * tanh(s / cap) before the softmax (arch/lib/transformer.json5:69-75);
        # 0: none.  Only the generic attention kernel applies one: with a cap the tensor-core kernels stand back.
        self.softcap = float(params.get("softcap", 0.0) or 0.0)
        names = ["q_proj"] if self.shares_kv else ["q_proj", "k_proj", "v_proj"]
        dtypes = {tensors[n + ".weight"].dtype for n in names}
        if len(dtypes) != 1:
            raise ValueError(f"q/k/v projections are stored in different dtypes: {sorted(map(str, dtypes))}")
        w = torch.cat([tensors[n + ".weight"] for n in names], 0)
        b = torch.cat([tensors[n + ".bias"].to(torch.float32) for n in names], 0) if params.get("bias") else None
        self.qkv = Linear(w, b, rt)
        self.out_proj = Linear(tensors["out_proj.weight"], tensors.get("out_proj.bias"), rt)
        f32 = lambda n: tensors[n].to(torch.float32).contiguous() if n in tensors else None
        self.q_gain, self.k_gain = f32("q_norm.weight"), f32("k_norm.weight")
        pos = params.get("position")
        self.position = None if pos is None else part_class("position", pos.kind)(pos.params, {}, rt)
        self.rotary = None if self.position is None else self.position.rotary()

    def kernel_libraries(self):
        return tuple(set(self.qkv.kernel_libraries()) | set(self.out_proj.kernel_libraries()) | {"core"})

    def cache_needs(self):
        return [] if self.shares_kv else [PagedKV(self.kv_heads, self.head_dim, self.window)]

    def attention_flops(self, n_tokens: int) -> int:
        """Scores and weighted values of a whole prompt over the causal half (or the
        window): 2 * 2 * head_dim multiply-adds per visible (query, key) pair and head."""
        pairs = n_tokens * (n_tokens + 1) // 2
        if self.window and n_tokens > self.window:
            pairs -= (n_tokens - self.window) * (n_tokens - self.window + 1) // 2
        return 4 * self.heads * self.head_dim * pairs

    def forward(self, h, residual, step, caches):
        kv = caches[0]
        if not self.shares_kv and not kv.writable:
            raise RuntimeError("an attention layer with k/v projections was given a read-only cache")
        qkv = self.qkv.partials(h)
        rot = self.rotary
        rope = (None if rot is None else rot.table, 0 if rot is None else rot.rotary_dim,
                False if rot is None else rot.adjacent_pairs)
        pages = (None if self.shares_kv else kv.k_pages, None if self.shares_kv else kv.v_pages)
        a = self.heads * self.head_dim
        if isinstance(qkv, ops.Partials):
            # K was split: this kernel adds the partial tiles itself (no reduction kernel in between)
            q = ops.qk_norm_rope_store_partials(
                qkv, self.rt.empty(qkv.shape[0], a), self.heads, self.kv_heads, self.head_dim, self.q_gain,
                self.k_gain, self.eps, *rope, step.tok_req, step.tok_pos, kv.block_table, *pages, step.status)
        else:
            ops.qk_norm_rope_store(qkv, self.heads, self.kv_heads, self.head_dim, self.q_gain, self.k_gain, self.eps,
                                   *rope, step.tok_req, step.tok_pos, kv.block_table, *pages, step.status)
            q = qkv[:, :a]
        out = self.rt.empty(qkv.shape[0], a)
        ops.paged_attention(q, self.heads, self.kv_heads, self.head_dim, kv.k_pages, kv.v_pages,
                            kv.block_table, step.tok_req, step.tok_pos, self.scale, self.window or 0, out,
                            step.status, hints=step, softcap=self.softcap)
        self.out_proj(out, out=residual, accumulate=True)

    def plan_ops(self, plan, h, caches):
        kv = caches[0]
        if not self.shares_kv and not kv.writable:
            raise RuntimeError("an attention layer with k/v projections was given a read-only cache")
        qkv = plan.linear(h, self.qkv.weight, self.qkv.bias, plan.buffer("qkv", self.qkv.out_features), "plain",
                          partials="always", role="qkv")
        plan.qk_norm_rope_store(qkv, self.heads, self.kv_heads, self.head_dim, self.q_gain, self.k_gain, self.eps,
                                self.rotary, kv, not self.shares_kv, plan.bt_stride)
        out = plan.attention(self.heads, self.kv_heads, self.head_dim, self.scale, self.window or 0, kv,
                             plan.bt_stride, softcap=self.softcap)
        plan.linear(out, self.out_proj.weight, self.out_proj.bias, None, "residual", role="out_proj")


register_part("mixer", "gqa_attention", GQAAttention)
