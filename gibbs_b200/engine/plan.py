"""A step's host work as data: the Python side of ``csrc/step_plan.cu``.

Running a model from Python costs a wrapper call, several tensor objects and
a ctypes call per kernel: some 15 microseconds each, about 2 ms for the 140
kernels of a step, more than the GPU needs for them.  Here every part of a
model appends its operations ONCE to a ``PlanBuilder`` (``plan_ops``: the
same work as its ``forward``, written as data), with activation buffers
allocated once for the largest step; a step is then one call into the C
library, which walks the list and launches the kernels.

The operations carry constants and *symbols*: the numbers and addresses that
change from step to step (tokens, requests, wanted rows, the longest portion
and context, the step's metadata, where the logits go).  A part that has no
``plan_ops`` (one written with tensor operations, say) makes the model "not
plannable": the engine then runs its ``forward`` methods as before.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..ops.library import KernelError, library
from ..parts.base import NotPlannable

OP = np.dtype([("op", "<i4"), ("flags", "<i4"), ("a", "<i8", (24,)), ("f", "<f8", (3,))])

P_EMBED, P_RMSNORM, P_LINEAR, P_SHORT_CONV, P_QKROPE, P_ATTENTION, P_SWIGLU, P_SCALE_SOFTCAP = range(1, 9)
LF_RESIDUAL, LF_PARTIALS_IF_ONE_EACH, LF_PARTIALS, LF_NORMED = 1, 2, 4, 8
NF_LAZY = 1

SYM_BIT = 1 << 62
(S_N, S_R, S_W, S_MAXQ, S_MAXCTX, S_ONE_EACH, S_TOKEN_IDS, S_TOK_REQ, S_TOK_POS, S_Q_START, S_Q_LEN, S_START_POS,
 S_CTX_LEN, S_SLOT_IDS, S_WANT_ROWS, S_LOGITS, S_BLOCK_TABLE0) = range(17)
S_TABLE_STRIDE = 31          # entries per request in the step's block tables
N_SYMBOLS = 32


def sym(index: int) -> int:
    return SYM_BIT | index


_FUNCTIONS = [("core", "gb_embed"), ("core", "gb_rmsnorm"), ("core", "gb_linear_simt"), ("tensorcore", "gb_linear_tc"),
              ("tensorcore", "gb_linear_tc_splits"), ("core", "gb_short_conv"), ("core", "gb_short_conv_partials"),
              ("core", "gb_qk_norm_rope_store"), ("core", "gb_qk_norm_rope_store_partials"),
              ("core", "gb_paged_attention"), ("tensorcore", "gb_attention_tc"), ("tensorcore", "gb_attention_tcgen05"),
              ("tensorcore", "gb_attention_tcgen05_supported"), ("core", "gb_swiglu"),
              ("tensorcore", "gb_linear_decode"), ("tensorcore", "gb_linear_decode_parts"),
              ("tensorcore", "gb_linear_decode_supported"), ("core", "gb_add_pending"),
              ("tensorcore", "gb_linear_decode_normed_ok"), ("core", "gb_scale_softcap")]


def register_op(name: str, function) -> int:
    """Make an operation of a part's own kernel library known to the step walker:
    ``function`` is a C function ``int f(const GbPlanCtx*, const long long* a, const
    double* f, int flags)`` (a ctypes function pointer, or its address) that launches the
    operation's kernels on ``ctx->stream`` and returns how many it launched.  Returns the
    id to pass to ``PlanBuilder.emit``."""
    lib = library("runtime")
    address = function if isinstance(function, int) else ctypes.cast(function, ctypes.c_void_p).value
    rc = lib.gb_plan_register_op(name.encode(), ctypes.c_void_p(address))
    if rc < 0:
        ops.check(lib, rc)
    return rc


class TableRef:
    """Stands for 'the block table of group g of the current step' while a plan is built."""

    def __init__(self, group: int):
        self.group = group


class SlotRef:
    """Stands for 'the slot ids of the current step'."""


class _Run(ctypes.Structure):
    _fields_ = [("ops", ctypes.c_void_p), ("n_ops", ctypes.c_int), ("sym", ctypes.c_void_p), ("n_sym", ctypes.c_int),
                ("ws", ctypes.c_void_p), ("attn_ws", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("attn_ctas", ctypes.c_int), ("tc_flags", ctypes.c_int), ("use_tcgen05", ctypes.c_int),
                ("defer_whole_rows", ctypes.c_int), ("failed_lib", ctypes.c_int), ("ssq", ctypes.c_void_p),
                ("decode_products", ctypes.c_int), ("residual", ctypes.c_void_p), ("residual_ld", ctypes.c_longlong),
                ("timing", ctypes.c_int), ("n_labels", ctypes.c_int), ("label_ms", ctypes.c_void_p),
                ("label_count", ctypes.c_void_p)]


class PlanBuilder:
    """Collects operations and owns the buffers they work on.  ``cap`` is the
    largest number of tokens a step may bring.  The residual stream is
    ``self.residual`` (float32 [cap, hidden]); a product that adds into it may
    leave partial sums for the next norm (the walker keeps track)."""

    def __init__(self, rt, hidden: int, cap: int, max_requests: int, with_tensorcore: bool):
        self.rt, self.device, self.hidden, self.cap = rt, rt.device, int(hidden), int(cap)
        self.max_requests = int(max_requests)
        self.tc = with_tensorcore
        self.ops: list = []
        self._buffers: dict = {}
        self._keep: list = []
        self.ws_floats = 1
        self.attn_ws_floats = 1
        self.ssq_floats = 1
        self._lazy = None           # (index of a norm's record, its output buffer): the next product may take it in
        self.labels: list = []      # names under which the operations' times are added up in timing mode
        self.bt_stride = 0
        self.LOGITS, self.WANTED = sym(S_LOGITS), S_W          # what a head writes to, and how many rows
        self.residual = self.buffer("residual", hidden, torch.float32)

    def buffer(self, name: str, width: int, dtype=None, rows: Optional[int] = None) -> torch.Tensor:
        """A [cap, width] buffer; the same name, width and dtype give the same buffer."""
        dtype = dtype or self.rt.dtype
        key = (name, int(width), dtype)
        t = self._buffers.get(key)
        if t is None:
            t = self._buffers[key] = torch.zeros(rows or self.cap, int(width), dtype=dtype, device=self.device)
        return t

    def keep(self, t: Optional[torch.Tensor]) -> int:
        """Device address of a tensor an operation reads (0 for None); the plan keeps it alive."""
        if t is None:
            return 0
        if not t.is_cuda:
            raise NotPlannable("a plan works on CUDA tensors")
        self._keep.append(t)
        return t.data_ptr()

    def emit(self, op: int, a, f=(), flags: int = 0, label: str = "") -> None:
        """Append one record: a built-in operation (P_...) or the id ``register_op`` gave.
        ``label``: the name its time is added up under in timing mode (operand 23 is kept for it)."""
        self._lazy = None
        if len(a) > 23:
            raise NotPlannable("an operation has 23 integer operands")
        label = label or f"op{op}"
        if label not in self.labels:
            self.labels.append(label)
        rec = np.zeros((), dtype=OP)
        rec["op"], rec["flags"] = op, flags
        rec["a"][:len(a)] = a
        rec["a"][23] = self.labels.index(label)
        rec["f"][:len(f)] = f
        self.ops.append(rec)

    # -- operations ------------------------------------------------------------
    def embed(self, table: torch.Tensor) -> None:
        if not table.is_contiguous() or table.shape[1] != self.hidden:
            raise NotPlannable("the embedding table must be contiguous [vocab, hidden]")
        self.emit(P_EMBED, [self.keep(table), ops.dtype_code(table.dtype), self.residual.data_ptr(), self.hidden,
                            table.shape[0]], label="embed")

    def rmsnorm(self, gain: torch.Tensor, eps: float, wanted_rows: bool = False, lazy: bool = False) -> torch.Tensor:
        """rmsnorm(residual (+ what the product before left to be added)) * gain; with
        ``wanted_rows`` only the step's wanted rows, gathered.  ``lazy``: the caller hands the
        result to ``linear`` next and nothing else reads it; steps of up to 64 rows then run
        the norm inside that product."""
        dim = self.hidden
        if gain.dtype != torch.float32 or gain.numel() != dim or not gain.is_contiguous():
            raise NotPlannable("a norm's gain is a contiguous float32 vector of the residual width")
        out = self.buffer("normed_wanted" if wanted_rows else "normed", dim)
        self.emit(P_RMSNORM, [self.residual.data_ptr(), dim, self.keep(gain), out.data_ptr(),
                              ops.dtype_code(out.dtype), int(wanted_rows), dim], [eps], label="rmsnorm")
        if lazy:
            self._lazy = (len(self.ops) - 1, out)
        return out

    def linear(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out, mode: str,
               rows_symbol: int = S_N, partials: str = "", role: str = "") -> torch.Tensor:
        """out (+)= x W^T + b.  mode: 'plain' (out in its own dtype), 'residual' (adds into the
        float32 residual; partial sums may be left to the next norm) or 'swiglu'.  ``partials``:
        '' | 'one_each' | 'always': when K is split, leave the partial tiles to the next
        operation (a short convolution or q/k kernel that adds them itself)."""
        n, k = weight.shape
        if x.shape[1] != k or weight.stride(1) != 1 or x.stride(1) != 1:
            raise NotPlannable("a product's operands have contiguous rows of equal length")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n or not bias.is_contiguous()):
            raise NotPlannable("a product's bias is a contiguous float32 vector")
        use_tc = (self.tc and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and k % 8 == 0
                  and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                  and weight.data_ptr() % 16 == 0)
        flags = 0
        lazy, self._lazy = self._lazy, None
        if lazy is not None and x is lazy[1] and use_tc and ops.DECODE_NORM_INSIDE and ops.linear_decode_supported(1, weight):
            self.ops[lazy[0]]["flags"] = int(self.ops[lazy[0]]["flags"]) | NF_LAZY
            self.ops[lazy[0]]["a"][7:9] = (n, k)
            flags |= LF_NORMED
        if mode == "residual":
            out, code = self.residual, 2
            flags |= LF_RESIDUAL
        elif mode == "swiglu":
            if not use_tc or n % 128 or out.dtype != torch.bfloat16:
                raise NotPlannable("the fused SwiGLU product runs on the tensor cores only")
            code = 3
        elif isinstance(out, int):
            code = 1                                                   # the step's float32 logits
        else:
            code = 0 if out.dtype == torch.bfloat16 else 1
            if partials and use_tc and out.dtype == torch.bfloat16:
                flags |= LF_PARTIALS if partials == "always" else LF_PARTIALS_IF_ONE_EACH
        if use_tc:
            # how K is split changes with the tile width (at 16, 32 and 64 rows) and then with
            # the number of 128-row tiles
            lib = library("tensorcore")
            for m in sorted({1, 17, 33, 65, 128, *range(256, self.cap + 128, 128)}):
                m = min(m, self.cap)
                s = lib.gb_linear_tc_splits(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
                if s > 1:
                    self.ws_floats = max(self.ws_floats, s * m * n)
            if mode == "residual":
                self.ws_floats = max(self.ws_floats, self.cap * n)     # large products are deferred whole
                if ops.linear_decode_supported(1, weight):
                    self.ssq_floats = max(self.ssq_floats, 64 * lib.gb_linear_decode_parts(ctypes.c_int(n),
                                                                                           ctypes.c_int(k)))
        self.emit(P_LINEAR, [x.data_ptr(), x.stride(0), self.keep(weight), weight.stride(0), self.keep(bias),
                             out if isinstance(out, int) else out.data_ptr(),
                             n if isinstance(out, int) else out.stride(0), sym(rows_symbol), n, k, 0 if use_tc else 1,
                             code, ops.dtype_code(x.dtype), ops.dtype_code(weight.dtype),
                             ops.F32 if isinstance(out, int) else ops.dtype_code(out.dtype)], flags=flags,
                  label="linear:" + (role or mode))
        return out

    def short_conv(self, bcx: torch.Tensor, taps: torch.Tensor, bias, slot_view, hidden: int, kernel: int):
        state = slot_view.state
        if not isinstance(slot_view.slot_ids, SlotRef) or state.dtype != torch.float32 \
                or state[0].stride() != (hidden, 1):
            raise NotPlannable("the short convolution keeps float32 state in the step's slots")
        out = self.buffer("mixed", hidden)
        self._keep.append(state)
        self.emit(P_SHORT_CONV, [bcx.data_ptr(), bcx.stride(0), self.keep(taps), self.keep(bias), state.data_ptr(),
                                 state.stride(0), out.data_ptr(), hidden, kernel, ops.dtype_code(bcx.dtype)],
                  label="short_conv")
        return out

    def qk_norm_rope_store(self, qkv: torch.Tensor, heads: int, kv_heads: int, hd: int, q_gain, k_gain, eps: float,
                           rotary, kv_view, write_kv: bool, bt_stride: int) -> None:
        if not isinstance(kv_view.block_table, TableRef):
            raise NotPlannable("attention reads the step's block tables")
        kp, vp = kv_view.k_pages, kv_view.v_pages
        q_out = self.buffer("q_rotated", heads * hd)
        self.emit(P_QKROPE,
                  [qkv.data_ptr(), qkv.stride(0), self.keep(q_gain), self.keep(k_gain),
                   self.keep(None if rotary is None else rotary.table), 0 if rotary is None else rotary.rotary_dim,
                   0 if rotary is None else int(rotary.adjacent_pairs), kv_view.block_table.group, kp.shape[2],
                   self.keep(kp) if write_kv else 0, self.keep(vp) if write_kv else 0, kp.shape[0] if write_kv else 0,
                   heads, kv_heads, hd, int(write_kv), ops.dtype_code(qkv.dtype), q_out.data_ptr(), bt_stride], [eps],
                  label="qk_rope")

    def attention(self, heads: int, kv_heads: int, hd: int, scale: float, window: int, kv_view, bt_stride: int,
                  softcap: float = 0.0):
        out = self.buffer("mixed", heads * hd)
        kp, vp = kv_view.k_pages, kv_view.v_pages
        # the decode kernel's key splits: every split leaves (head_dim + 2) floats per (token, head); a
        # request brings at most 16 // group tokens to that kernel, and the more requests the fewer splits
        group = max(1, heads // kv_heads)
        per_request = max(1, 16 // group) * heads * (hd + 2)
        need = max(ops.attention_splits(n, kv_heads, 1 << 30) * n * per_request
                   for n in range(1, self.max_requests + 1))
        self.attn_ws_floats = max(self.attn_ws_floats, need)
        self.emit(P_ATTENTION, [out.data_ptr(), out.stride(0), self.keep(kp), self.keep(vp), kv_view.block_table.group,
                                kp.shape[2], kp.shape[0], heads, kv_heads, hd, int(window or 0),
                                ops.dtype_code(out.dtype), bt_stride], [scale, softcap], label="attention")
        return out

    def scale_softcap(self, values: int, columns: int, rows_symbol: int, scale: float, cap: float) -> None:
        """values <- values * scale, then cap * tanh(values / cap) when cap > 0; ``values`` is a
        symbol (the step's logits) or an address, [rows, columns] float32."""
        self.emit(P_SCALE_SOFTCAP, [values, columns, sym(rows_symbol)], [scale, cap], label="scale_softcap")

    def swiglu(self, gate_up: torch.Tensor, inner: int) -> torch.Tensor:
        out = self.buffer("act", inner)
        self.emit(P_SWIGLU, [gate_up.data_ptr(), out.data_ptr(), ops.dtype_code(out.dtype), inner], label="swiglu")
        return out


class StepPlan:
    """A finished plan: the operation list (host memory, read by the C walker), its buffers,
    and ``run``."""

    _bound = None      # None: nothing bound yet; False: the core library only; True: the tensor-core library as well

    def __init__(self, b: PlanBuilder, n_groups: int):
        self.lib = library("runtime")
        self._bind(b.tc)
        self.table = np.stack(b.ops) if b.ops else np.zeros(0, dtype=OP)
        if self.table.dtype.itemsize != self.lib.gb_plan_op_bytes():
            raise KernelError("the plan's record layout does not match the library")
        self.device = b.device
        self._keep = (b._keep, b._buffers)
        self.ws = torch.empty(b.ws_floats, dtype=torch.float32, device=b.device)
        self.attn_ws = torch.empty(b.attn_ws_floats, dtype=torch.float32, device=b.device)
        self.ssq = torch.empty(b.ssq_floats, dtype=torch.float32, device=b.device)
        self.symbols = np.zeros(N_SYMBOLS, dtype=np.int64)
        self.n_groups = n_groups
        self.cap, self.max_requests = b.cap, b.max_requests
        r = self._run = _Run()
        r.ops, r.n_ops = self.table.ctypes.data, len(self.table)
        r.sym, r.n_sym = self.symbols.ctypes.data, N_SYMBOLS
        r.ws, r.attn_ws = self.ws.data_ptr(), self.attn_ws.data_ptr()
        r.status = ops.device_status(b.device).data_ptr()
        r.attn_ctas, r.tc_flags, r.use_tcgen05 = ops._ATTN_CTAS, ops._TC_FLAGS, int(ops._ATTN_TCGEN05)
        r.defer_whole_rows = ops.DEFER_WHOLE_ROWS
        r.ssq, r.decode_products = self.ssq.data_ptr(), (ops.DECODE_ROWS if b.tc else 0)
        r.residual, r.residual_ld = b.residual.data_ptr(), b.residual.stride(0)
        self.labels = list(b.labels)
        self.label_ms = np.zeros(max(len(self.labels), 1), dtype=np.float32)
        self.label_count = np.zeros(max(len(self.labels), 1), dtype=np.int32)
        r.timing, r.n_labels = 0, len(self.labels)
        r.label_ms, r.label_count = self.label_ms.ctypes.data, self.label_count.ctypes.data

    def set_timing(self, on: bool) -> None:
        """Timing mode: the walker brackets every operation with CUDA events, waits for the step
        and adds each operation's time to its label (see ``timing_table``).  Operations then run
        one after the other, so the times are those of kernels that do not overlap: good for
        shares, not for the step's own duration.  Not for use inside a CUDA graph."""
        self._run.timing = 1 if on else 0
        self.label_ms[:] = 0
        self.label_count[:] = 0

    def timing_table(self) -> dict:
        """{label: (operations timed, milliseconds in total)} since ``set_timing(True)``."""
        return {name: (int(self.label_count[i]), float(self.label_ms[i])) for i, name in enumerate(self.labels)
                if self.label_count[i]}

    def _bind(self, need_tensorcore: bool) -> None:
        """Hand the walker the entry points of the kernel libraries; those of the tensor-core
        library only once a model needs it (a float32 model never builds that library)."""
        if StepPlan._bound is True or (StepPlan._bound is False and not need_tensorcore):
            return
        fns = (ctypes.c_void_p * len(_FUNCTIONS))()
        for i, (lib_name, fn) in enumerate(_FUNCTIONS):
            if lib_name == "tensorcore" and not need_tensorcore:
                fns[i] = None
            else:
                fns[i] = ctypes.cast(getattr(library(lib_name), fn), ctypes.c_void_p).value
        rc = self.lib.gb_plan_bind(fns, ctypes.c_int(len(_FUNCTIONS)))
        if rc != 0:
            ops.check(self.lib, rc)
        StepPlan._bound = bool(need_tensorcore)

    def run(self, n_tokens: int, n_requests: int, n_want: int, max_q_len: int, max_ctx_len: int, meta_ptr: int, offs,
            mb: int, logits_ptr: int) -> int:
        """Launch one step whose metadata lies at ``meta_ptr`` (int32 words at ``offs``, as the
        step builder lays them out; ``mb`` entries per request in a block table)."""
        s = self.symbols
        s[S_N], s[S_R], s[S_W], s[S_MAXQ], s[S_MAXCTX] = n_tokens, n_requests, n_want, max_q_len, max_ctx_len
        s[S_ONE_EACH] = 1 if (max_q_len == 1 and n_tokens == n_requests) else 0
        for k, i in ((S_TOKEN_IDS, 0), (S_TOK_REQ, 1), (S_TOK_POS, 2), (S_Q_START, 3), (S_Q_LEN, 4), (S_START_POS, 5),
                     (S_CTX_LEN, 6), (S_SLOT_IDS, 7), (S_WANT_ROWS, 8)):
            s[k] = meta_ptr + 4 * offs[i]
        s[S_LOGITS] = logits_ptr
        s[S_TABLE_STRIDE] = mb
        for g in range(self.n_groups):
            s[S_BLOCK_TABLE0 + g] = meta_ptr + 4 * (offs[9] + g * n_requests * mb)
        rc = self.lib.gb_plan_run(ctypes.byref(self._run), ops._STREAM if ops._STREAM is not None else ops._stream())
        if rc < 0:
            which = self._run.failed_lib
            ops.check(self.lib if which == 2 else library("tensorcore" if which == 1 else "core"), rc)
        ops._launched(rc)
        return rc


def build_step_plan(model, cache, cap: int, max_requests: int) -> StepPlan:
    """The plan of ``model`` over ``cache`` for steps of up to ``cap`` tokens.  Raises
    NotPlannable if some part of the model cannot be written as operations."""
    if len(cache.groups) > S_TABLE_STRIDE - S_BLOCK_TABLE0:
        raise NotPlannable(f"{len(cache.groups)} cache groups")
    with_tc = "tensorcore" in model.kernel_libraries()
    b = PlanBuilder(model.rt, model.hidden_size, cap, max_requests, with_tc)
    b.bt_stride = sym(S_TABLE_STRIDE)          # a step packs only as many table columns as its longest context needs
    views = cache.views([TableRef(g) for g in range(len(cache.groups))], SlotRef(), [])
    model.plan_ops(b, views)
    return StepPlan(b, len(cache.groups))


ENABLED = os.environ.get("GIBBS_B200_PLAN", "1") != "0"
