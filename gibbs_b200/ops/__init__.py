"""Python bindings of the hand-written CUDA kernels.

Every function takes CUDA tensors, checks what the kernel assumes (device,
dtype, contiguous rows) and launches on the current CUDA stream.  Nothing
here computes on the host or calls a library kernel: if a tensor is not on a
GPU or a kernel library is missing, the call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .library import KernelError, check, ensure_built, library

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_c_int, _c_ll, _c_float, _c_void = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


_LAUNCHES = 0
_LIBS: dict = {}        # kernel libraries already loaded, by name


def _lib(name: str):
    lib = _LIBS[name] = library(name)
    return lib


def _launched(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launch_count() -> int:
    """Kernels of this package launched so far in this process (each wrapper
    adds the number of kernels its call enqueues)."""
    return _LAUNCHES


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]):
    return _c_void(t.data_ptr()) if t is not None else _c_void(0)


_STREAM = None      # handle of the stream kernels launch on while a `launching_on` block is active


def _stream():
    if _STREAM is not None:
        return _STREAM
    return _c_void(torch.cuda.current_stream().cuda_stream)


class launching_on:
    """Within the block every kernel of this module launches on ``stream`` (default: the
    current CUDA stream at entry) without asking torch for the current stream at every
    launch, which costs more than the launch itself.  The caller must not switch streams
    inside the block."""

    def __init__(self, stream=None):
        self.stream = stream

    def __enter__(self):
        global _STREAM
        self.prev = _STREAM
        st = self.stream if self.stream is not None else torch.cuda.current_stream()
        _STREAM = _c_void(st.cuda_stream)
        return self

    def __exit__(self, *exc):
        global _STREAM
        _STREAM = self.prev


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("gibbs_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride (in elements) of a 2-d tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: expected a 2-d tensor with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _i32(t: Optional[torch.Tensor], what: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what}: expected a contiguous int32 tensor")
    return t


def _f32vec(t: Optional[torch.Tensor], n: int, what: str):
    if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n):
        raise KernelError(f"{what}: expected {n} contiguous float32 values, got {tuple(t.shape)} {t.dtype}")
    return t


# ---------------------------------------------------------------------------

def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] widened to 32-bit."""
    _need_cuda(table, ids, out)
    lib = library("core")
    n, dim = out.shape
    if not table.is_contiguous() or table.shape[1] != dim or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("embed: table [vocab, dim] contiguous and out [n, dim] float32 contiguous expected")
    _i32(ids, "embed ids")
    _launched(1)
    check(lib, lib.gb_embed(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), _c_int(n), _c_int(dim),
                            _c_int(table.shape[0]), _stream()))
    return out


def feed_tokens(ids: torch.Tensor, picked: torch.Tensor, source: torch.Tensor) -> torch.Tensor:
    """ids[t] = picked[source[t]] wherever source[t] >= 0 (all int32, on the device)."""
    _need_cuda(ids, picked, source)
    lib = library("core")
    for t, what in ((ids, "feed_tokens ids"), (picked, "feed_tokens picked"), (source, "feed_tokens source")):
        _i32(t, what)
    if source.numel() != ids.numel():
        raise KernelError("feed_tokens: one source index per token id expected")
    _launched(1)
    check(lib, lib.gb_feed_tokens(_ptr(ids), _ptr(picked), _ptr(source), _c_int(ids.numel()),
                                  _c_int(picked.numel()), _stream()))
    return ids


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, pending=None) -> torch.Tensor:
    """out[r, :] = x[rows[r] or r, :] * rsqrt(mean(x^2) + eps) * gain; x is 32-bit.
    ``pending`` = (partials [splits, n, dim], bias or None): sums a split-K
    product left to be added to x first (and, without ``rows``, written back)."""
    lib = _LIBS.get("core") or _lib("core")
    n_x, dim = x.shape
    if not (x.is_cuda and gain.is_cuda and out.is_cuda):
        _need_cuda(x, gain, out)
    if x.dtype != torch.float32:
        raise KernelError("rmsnorm: the input (the residual stream) is float32")
    if dim > 1 and x.stride(1) != 1:
        raise KernelError("rmsnorm x: expected a 2-d tensor with contiguous rows")
    n_rows = out.shape[0]
    if not out.is_contiguous() or out.shape[1] != dim:
        raise KernelError("rmsnorm: out must be contiguous [rows, dim]")
    if rows is None:
        if n_rows != n_x:
            raise KernelError("rmsnorm: out has a different number of rows than x")
    else:
        _need_cuda(rows)
        _i32(rows, "rmsnorm rows")
    if gain.dtype != torch.float32 or gain.numel() != dim or not gain.is_contiguous():
        _f32vec(gain, dim, "rmsnorm gain")
    odt = out.dtype
    if odt == torch.bfloat16:
        code = BF16
    elif odt == torch.float32:
        code = F32
    else:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {odt}")
    ws = pbias = None
    splits = 0
    if pending is not None:
        ws, pbias = pending
        splits = ws.shape[0]
        if ws.dtype != torch.float32 or not ws.is_contiguous() or ws.shape[1:] != x.shape:
            raise KernelError("rmsnorm: pending partial sums must be contiguous float32 [splits, n, dim]")
        if pbias is not None:
            _need_cuda(pbias)
            _f32vec(pbias, dim, "rmsnorm pending bias")
    _launched(1)
    rc = lib.gb_rmsnorm(_c_void(x.data_ptr()), _c_ll(x.stride(0) if n_x > 1 else max(x.stride(0), dim)),
                        _c_void(gain.data_ptr()), _c_void(out.data_ptr()), _c_int(code),
                        _NULL if rows is None else _c_void(rows.data_ptr()), _c_int(n_rows), _c_int(dim), _c_float(eps),
                        _NULL if ws is None else _c_void(ws.data_ptr()), _c_int(splits), _c_ll(n_x),
                        _NULL if pbias is None else _c_void(pbias.data_ptr()),
                        _STREAM if _STREAM is not None else _stream())
    if rc:
        check(lib, rc)
    return out


def add_pending(x: torch.Tensor, ws: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """x += sum over splits of ws[s] (+ bias), in split order."""
    _need_cuda(x, ws, bias)
    lib = library("core")
    if x.dtype != torch.float32 or ws.dtype != torch.float32 or not ws.is_contiguous() or ws.shape[1:] != x.shape:
        raise KernelError("add_pending: x float32 [n, dim] and partial sums float32 [splits, n, dim] expected")
    _f32vec(bias, x.shape[1], "add_pending bias")
    _launched(1)
    check(lib, lib.gb_add_pending(_ptr(x), _c_ll(_rows(x, "x")), _ptr(ws), _c_int(ws.shape[0]), _ptr(bias),
                                  _c_ll(x.shape[0]), _c_int(x.shape[1]), _stream()))
    return x


def linear_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias) with 32-bit FMA on the CUDA cores."""
    _need_cuda(a, w, bias, out)
    lib = library("core")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelError(f"linear: shapes a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} disagree")
    _f32vec(bias, n, "linear bias")
    _launched(1)
    check(lib, lib.gb_linear_simt(
        _ptr(a), dtype_code(a.dtype), _c_ll(_rows(a, "linear a")), _ptr(w), dtype_code(w.dtype),
        _c_ll(_rows(w, "linear w")), _ptr(bias), _ptr(out), dtype_code(out.dtype), _c_ll(_rows(out, "linear out")),
        _c_int(1 if accumulate else 0), _c_int(m), _c_int(n), _c_int(k), _stream()))
    return out


def linear_libraries(weight_dtype: torch.dtype, compute_dtype: torch.dtype):
    """Kernel libraries a projection with these operand types launches from."""
    if weight_dtype == torch.bfloat16 and compute_dtype == torch.bfloat16:
        return ("core", "tensorcore")
    return ("core",)


_STATUS: dict = {}
_SPLITS: dict = {}      # (m, n, k) -> number of K splits the tensor-core product uses


def device_status(device) -> torch.Tensor:
    """The int32 word of ``device`` that kernels set when a bounded wait ran
    out or a page id was outside its pool (0: nothing happened)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _STATUS.get(key)
    if t is None:
        t = _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS_PTR[key] = _c_void(t.data_ptr())
    return t


_STATUS_PTR: dict = {}
_NULL, _ZERO, _ONE = _c_void(0), _c_int(0), _c_int(1)


def _status_ptr(t: torch.Tensor):
    """The status word of the device ``t`` lives on, as a C pointer."""
    p = _STATUS_PTR.get(t.device.index)
    return p if p is not None else _c_void(device_status(t.device).data_ptr())


# tuning switch of the tensor-core product: evict-first hint on the weights of decode-sized products
_TC_FLAGS = 1 if os.environ.get("GIBBS_B200_EVICT_FIRST", "1") != "0" else 0


# From this many rows on, a product that adds into the 32-bit residual stream does not read and
# rewrite the stream from its epilogue: it stores its result as one set of "partial" tiles, which
# the norm that reads the stream next adds (measured on 2,048-token prompts: the read-modify-write
# epilogue was what those products waited for).  The step walker (csrc/step_plan.cu) has the same rule.
DEFER_WHOLE_ROWS = 256


def linear_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              accumulate: bool = False, swiglu: bool = False, defer: bool = False):
    """out (+)= a @ w.T (+ bias) for bfloat16 a and w on the tensor cores
    (csrc/gemm_tc.cu).  ``swiglu``: w holds gate and up rows alternating in
    blocks of 64 and out [m, n/2] gets (g * sigmoid(g)) * u.
    ``defer`` (with ``accumulate``, or for a plain bfloat16 product): when
    the kernel splits K, nothing is written to ``out``; the partial sums
    [splits, m, n] are returned instead, for the caller's next kernel to add
    (without the bias).  Otherwise returns ``out``."""
    # (this wrapper runs some seventy times a step: its checks are the cheap ones)
    lib = _LIBS.get("tensorcore") or _lib("tensorcore")
    m, k = a.shape
    n, kw = w.shape
    n_out = n // 2 if swiglu else n
    if not (a.is_cuda and w.is_cuda and out.is_cuda):
        _need_cuda(a, w, out)
    if kw != k or out.shape[0] != m or out.shape[1] != n_out:
        raise KernelError(f"linear: shapes a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} disagree")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("linear_tc: bfloat16 operands expected")
    if a.stride(1) != 1 or w.stride(1) != 1 or (n_out > 1 and out.stride(1) != 1):
        raise KernelError("linear: expected 2-d tensors with contiguous rows")
    odt = out.dtype
    if swiglu:
        if odt != torch.bfloat16 or n % 128:
            raise KernelError("linear_tc: the SwiGLU epilogue writes bfloat16 and needs 2*features % 128 == 0")
        mode = 3
    elif accumulate:
        if odt != torch.float32:
            raise KernelError("linear_tc: accumulation needs a float32 output")
        mode = 2
    elif odt == torch.bfloat16:
        mode = 0
    elif odt == torch.float32:
        mode = 1
    else:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {odt}")
    if bias is not None:
        _need_cuda(bias)
        _f32vec(bias, n, "linear bias")
    key = (m, n, k)
    splits = _SPLITS.get(key)
    if splits is None:
        splits = _SPLITS[key] = lib.gb_linear_tc_splits(_c_int(m), _c_int(n), _c_int(k))
    # a large unsplit product into the residual stream is deferred as a whole (see DEFER_WHOLE_ROWS)
    whole = bool(defer and accumulate and splits == 1 and m >= DEFER_WHOLE_ROWS)
    ws = torch.empty((splits, m, n), dtype=torch.float32, device=a.device) if (splits > 1 or whole) else None
    defer = bool(defer and (accumulate or mode == 0) and splits > 1) or whole
    rc = lib.gb_linear_tc(
        _c_void(a.data_ptr()), _c_ll(a.stride(0) if m > 1 else max(a.stride(0), k)), _c_void(w.data_ptr()),
        _c_ll(w.stride(0) if n > 1 else max(w.stride(0), k)), _NULL if bias is None else _c_void(bias.data_ptr()),
        _c_void(out.data_ptr()), _c_int(mode), _c_ll(out.stride(0) if m > 1 else max(out.stride(0), n_out)), _c_int(m),
        _c_int(n), _c_int(k), _NULL if ws is None else _c_void(ws.data_ptr()),
        _c_int(2) if whole else (_ONE if defer else _ZERO),
        _c_int(_TC_FLAGS),
        _status_ptr(a), _STREAM if _STREAM is not None else _stream())
    if rc < 0:
        check(lib, rc)
    _launched(rc)
    return ws if defer else out


# Products of up to this many rows run on the cluster kernel (csrc/gemm_tc_decode.cu, which takes up to 64:
# K split inside a thread-block cluster, the norm in front of a product inside it for up to 16 rows).
# 0 (the default): all products on the general kernel, whose split-K partial tiles the next kernel adds.
# Measured on a B200 at batch 8, 2,048-token contexts: 0.835 ms a step by default, 0.918 ms with the
# cluster kernel and the norms as kernels of their own, 1.07 ms with the norms inside the products (the
# exchange through distributed shared memory and the cluster barrier cost every product about 2 us more
# than a partial tile costs its consumer, and normalising the rows in every CTA costs more instructions
# on the critical path than the norm kernel's launch).
DECODE_ROWS = max(0, min(64, int(os.environ.get("GIBBS_B200_DECODE_ROWS", "0"))))
DECODE_PRODUCTS = DECODE_ROWS > 0
# 0: the norm in front of a decode product stays a kernel of its own (for comparison)
DECODE_NORM_INSIDE = os.environ.get("GIBBS_B200_DECODE_NORM_INSIDE", "1") != "0"


def linear_decode_supported(m: int, w: torch.Tensor) -> bool:
    """Whether ``linear_decode`` takes a product of ``m`` rows with this weight."""
    return (1 <= m <= 64 and w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.shape[1] % 8 == 0
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)


def linear_decode_normed_ok(m: int, n: int, k: int) -> bool:
    """Whether a decode product of these sizes can run the norm of its rows itself."""
    lib = _LIBS.get("tensorcore") or _lib("tensorcore")
    return bool(lib.gb_linear_decode_normed_ok(_c_int(m), _c_int(n), _c_int(k)))


class NormedRows:
    """Rows of the 32-bit residual stream that a product is to read through an
    RMSNorm: ``x`` float32 [n, dim], ``gain``, ``eps``; ``rows`` (int32, optional)
    picks and orders the rows; ``ssq`` (optional) are partial sums of squares
    [parts, n] of the rows of ``x``, as a product into the stream left them."""

    def __init__(self, x: torch.Tensor, gain: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                 ssq: Optional[torch.Tensor] = None):
        self.x, self.gain, self.eps, self.rows, self.ssq = x, gain, float(eps), rows, ssq
        self.n_rows = x.shape[0] if rows is None else rows.numel()
        self.shape = (self.n_rows, x.shape[1])
        self.device, self.dtype = x.device, torch.bfloat16

    def tensor(self) -> torch.Tensor:
        """The normalised rows as a bfloat16 tensor (the norm as a kernel of its own)."""
        out = torch.empty(self.shape, dtype=torch.bfloat16, device=self.x.device)
        return rmsnorm(self.x, self.gain, self.eps, out, self.rows)


_PARTS: dict = {}       # (n, k) -> partial sums of squares per row a product into the stream leaves


def linear_decode(a, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, accumulate: bool = False,
                  swiglu: bool = False, want_ssq: bool = False):
    """out (+)= a @ w.T (+ bias) for up to 64 rows (csrc/gemm_tc_decode.cu): K is
    split inside a thread-block cluster and added through distributed shared
    memory, so nothing but ``out`` is written.  ``a`` is a bfloat16 tensor, or
    ``NormedRows`` (the RMSNorm then runs inside the product).  With
    ``accumulate`` and ``want_ssq`` the partial sums of squares of the new rows
    of ``out`` are returned ([parts, m] float32), else None."""
    lib = _LIBS.get("tensorcore") or _lib("tensorcore")
    normed = isinstance(a, NormedRows)
    m, k = a.shape
    n, kw = w.shape
    n_out = n // 2 if swiglu else n
    if kw != k or out.shape[0] != m or out.shape[1] != n_out:
        raise KernelError(f"linear: shapes a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} disagree")
    if not linear_decode_supported(m, w):
        raise KernelError("linear_decode: 1 to 64 rows and a bfloat16 weight with 16-byte aligned rows expected")
    if n_out > 1 and out.stride(1) != 1:
        raise KernelError("linear: expected 2-d tensors with contiguous rows")
    odt = out.dtype
    if swiglu:
        if odt != torch.bfloat16 or n % 128:
            raise KernelError("linear_decode: the SwiGLU epilogue writes bfloat16 and needs 2*features % 128 == 0")
        mode = 3
    elif accumulate:
        if odt != torch.float32:
            raise KernelError("linear_decode: accumulation needs a float32 output")
        mode = 2
    elif odt == torch.bfloat16:
        mode = 0
    elif odt == torch.float32:
        mode = 1
    else:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {odt}")
    if bias is not None:
        _need_cuda(bias)
        _f32vec(bias, n, "linear bias")
    gain = rows = ssq_in = _NULL
    eps, parts_in, ld_in = 0.0, 0, 0
    if normed:
        x = a.x
        _need_cuda(x, a.gain, a.rows, a.ssq, w, out)
        if x.dtype != torch.float32 or x.stride(1) != 1 or x.stride(0) % 4 or x.data_ptr() % 16:
            raise KernelError("linear_decode: normalised rows are float32 with 16-byte aligned rows")
        _f32vec(a.gain, k, "rmsnorm gain")
        gain, eps = _c_void(a.gain.data_ptr()), a.eps
        if a.rows is not None:
            rows = _c_void(_i32(a.rows, "rmsnorm rows").data_ptr())
        if a.ssq is not None:
            if a.ssq.dtype != torch.float32 or not a.ssq.is_contiguous() or a.ssq.shape[1] != x.shape[0]:
                raise KernelError("linear_decode: partial sums of squares are contiguous float32 [parts, rows of x]")
            ssq_in, parts_in, ld_in = _c_void(a.ssq.data_ptr()), a.ssq.shape[0], a.ssq.shape[1]
        ldx = x.stride(0) if x.shape[0] > 1 else max(x.stride(0), k)
    else:
        x = a
        if not (x.is_cuda and w.is_cuda and out.is_cuda):
            _need_cuda(x, w, out)
        if x.dtype != torch.bfloat16 or x.stride(1) != 1:
            raise KernelError("linear_decode: bfloat16 rows expected")
        ldx = x.stride(0) if m > 1 else max(x.stride(0), k)
    ssq = None
    if want_ssq and mode == 2:
        parts = _PARTS.get((n, k))
        if parts is None:
            parts = _PARTS[(n, k)] = lib.gb_linear_decode_parts(_c_int(n), _c_int(k))
        ssq = torch.empty((parts, m), dtype=torch.float32, device=out.device)
    rc = lib.gb_linear_decode(
        _c_void(x.data_ptr()), _c_ll(ldx), _c_int(1 if normed else 0), gain, _c_float(eps), rows, ssq_in,
        _c_int(parts_in), _c_ll(ld_in), _c_void(w.data_ptr()), _c_ll(w.stride(0) if n > 1 else max(w.stride(0), k)),
        _NULL if bias is None else _c_void(bias.data_ptr()), _c_void(out.data_ptr()), _c_int(mode),
        _c_ll(out.stride(0) if m > 1 else max(out.stride(0), n_out)), _c_int(m), _c_int(n), _c_int(k),
        _NULL if ssq is None else _c_void(ssq.data_ptr()), _c_ll(m), _c_int(_TC_FLAGS), _status_ptr(out),
        _STREAM if _STREAM is not None else _stream())
    if rc < 0:
        check(lib, rc)
    _launched(rc)
    return ssq


class Partials:
    """What a split-K product left for its consumer: the 32-bit partial tiles
    [splits, m, n] (to be added in split order), the product's bias (not yet
    added) or None, and the dtype the sum is to be rounded to."""

    def __init__(self, ws: torch.Tensor, bias: Optional[torch.Tensor], dtype: torch.dtype):
        self.ws, self.bias, self.dtype = ws, bias, dtype
        self.shape = tuple(ws.shape[1:])


def linear_tc_partials(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]):
    """a @ w.T on the tensor cores for a consumer that can add split-K partial
    tiles itself: returns ``Partials`` when the kernel splits K for these sizes
    (no reduction kernel runs), else the finished bfloat16 product."""
    m, n = a.shape[0], w.shape[0]
    out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    res = linear_tc(a, w, bias, out, defer=True)
    return Partials(res, bias, torch.bfloat16) if res is not out else out


def linear_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    k = a.shape[1]
    return (k % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
           accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias); picks the matrix-product kernel for the
    operand types: tensor cores for bfloat16 x bfloat16, 32-bit FMA otherwise
    (float32 operands, a weight kept in 32-bit, rows TMA cannot address)."""
    if linear_tc_supported(a, w):
        return linear_tc(a, w, bias, out, accumulate)
    return linear_simt(a, w, bias, out, accumulate)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = (g * sigmoid(g)) * u for rows [g | u]."""
    _need_cuda(gate_up, out)
    lib = library("core")
    n, inner = out.shape
    if gate_up.shape != (n, 2 * inner) or not gate_up.is_contiguous() or not out.is_contiguous() \
            or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: gate_up [n, 2*inner] and out [n, inner], contiguous, same dtype expected")
    _launched(1)
    check(lib, lib.gb_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), _c_int(n), _c_int(inner), _stream()))
    return out


def cast(src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need_cuda(src, out)
    lib = library("core")
    if not src.is_contiguous() or not out.is_contiguous() or src.numel() != out.numel():
        raise KernelError("cast: contiguous tensors of equal size expected")
    _launched(1)
    check(lib, lib.gb_cast(_ptr(src), dtype_code(src.dtype), _ptr(out), dtype_code(out.dtype),
                           _c_ll(src.numel()), _stream()))
    return out


def short_conv(bcx: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               slot_ids: torch.Tensor, tok_req: torch.Tensor, q_start: torch.Tensor, q_len: torch.Tensor,
               out: torch.Tensor, max_q_len: int = 0) -> torch.Tensor:
    """Gated short convolution over a ragged batch; see csrc/conv.cu.
    state: float32 [n_slots, kernel-1, hidden] (the slot axis may be strided)."""
    _need_cuda(bcx, taps, bias, state, slot_ids, tok_req, q_start, q_len, out)
    lib = library("core")
    n, hidden = out.shape
    kk = taps.shape[1]
    if bcx.shape != (n, 3 * hidden) or bcx.dtype != out.dtype or not out.is_contiguous():
        raise KernelError("short_conv: bcx [n, 3*hidden] and out [n, hidden] of one dtype expected")
    _f32vec(taps, hidden * kk, "short_conv taps")
    _f32vec(bias, hidden, "short_conv bias")
    if state.dtype != torch.float32 or state.shape[1:] != (kk - 1, hidden) or state[0].stride() != (hidden, 1):
        raise KernelError(f"short_conv: state must be float32 [slots, {kk - 1}, {hidden}] with contiguous slots")
    for t, w in ((slot_ids, "slot_ids"), (tok_req, "tok_req"), (q_start, "q_start"), (q_len, "q_len")):
        _i32(t, "short_conv " + w)
    rc = lib.gb_short_conv(
        _ptr(bcx), dtype_code(bcx.dtype), _c_ll(_rows(bcx, "short_conv bcx")), _ptr(taps), _ptr(bias), _ptr(state),
        _c_ll(state.stride(0)), _ptr(slot_ids), _ptr(tok_req), _ptr(q_start), _ptr(q_len), _ptr(out), _c_int(n),
        _c_int(q_len.numel()), _c_int(hidden), _c_int(kk), _c_int(max_q_len), _stream())
    if rc < 0:
        check(lib, rc)
    _launched(rc)
    return out


def short_conv_partials(bcx: Partials, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                        slot_ids: torch.Tensor, q_start: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """The gated short convolution of one token per request, reading [B | C | x]
    as the partial tiles of the product that made it (no reduction kernel in between)."""
    _need_cuda(bcx.ws, bcx.bias, taps, bias, state, slot_ids, q_start, out)
    lib = library("core")
    n, hidden = out.shape
    kk = taps.shape[1]
    ws = bcx.ws
    if ws.dtype != torch.float32 or not ws.is_contiguous() or ws.shape[1:] != (n, 3 * hidden) \
            or out.dtype != torch.bfloat16 or not out.is_contiguous() or bcx.dtype != torch.bfloat16:
        raise KernelError("short_conv_partials: partial tiles [splits, n, 3*hidden] float32 and out [n, hidden] "
                          "bfloat16 expected")
    if q_start.numel() != n:
        raise KernelError("short_conv_partials: one token per request expected")
    _f32vec(taps, hidden * kk, "short_conv taps")
    _f32vec(bias, hidden, "short_conv bias")
    _f32vec(bcx.bias, 3 * hidden, "short_conv in_proj bias")
    if state.dtype != torch.float32 or state.shape[1:] != (kk - 1, hidden) or state[0].stride() != (hidden, 1):
        raise KernelError(f"short_conv: state must be float32 [slots, {kk - 1}, {hidden}] with contiguous slots")
    _i32(slot_ids, "short_conv slot_ids"), _i32(q_start, "short_conv q_start")
    rc = lib.gb_short_conv_partials(
        _ptr(ws), _c_int(ws.shape[0]), _c_ll(n), _ptr(bcx.bias), _ptr(taps), _ptr(bias), _ptr(state),
        _c_ll(state.stride(0)), _ptr(slot_ids), _ptr(q_start), _ptr(out), _c_int(n), _c_int(hidden), _c_int(kk),
        _stream())
    if rc < 0:
        check(lib, rc)
    _launched(rc)
    return out


def _rotary_table(inv_freq: Optional[torch.Tensor], rotary_dim: int) -> Optional[torch.Tensor]:
    """The table the rotary kernels read: rotary_dim / 2 frequencies followed by the factor on
    cosines and sines.  Frequencies alone get the factor 1 appended (``parts.base.Rotary``
    hands over the finished table)."""
    if inv_freq is None:
        return None
    half = rotary_dim // 2
    if inv_freq.numel() == half:
        return torch.cat([inv_freq.to(torch.float32).reshape(-1), torch.ones(1, dtype=torch.float32, device=inv_freq.device)])
    return _f32vec(inv_freq, half + 1, "rotary table")


def _check_pages(k_pages, v_pages, kv_heads, hd, dtype, what):
    for p in (k_pages, v_pages):
        if p.dim() != 4 or p.shape[1] != kv_heads or p.shape[3] != hd or not p.is_contiguous() or p.dtype != dtype:
            raise KernelError(f"{what}: pages must be contiguous [n_pages, {kv_heads}, page_size, {hd}] {dtype}, "
                              f"got {tuple(p.shape)} {p.dtype}")
    if k_pages.shape != v_pages.shape:
        raise KernelError(f"{what}: key and value pages differ in shape")


def qk_norm_rope_store(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                       q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], rotary_dim: int, adjacent_pairs: bool,
                       tok_req: torch.Tensor, tok_pos: torch.Tensor, block_table: torch.Tensor,
                       k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                       status: torch.Tensor) -> None:
    """Per-head RMSNorm and rotary encoding of q (in place) and k; k and v go
    into their pages.  With k_pages None only q is processed (a layer that
    reads another layer's cache)."""
    _need_cuda(qkv, q_gain, k_gain, inv_freq, tok_req, tok_pos, block_table, k_pages, v_pages, status)
    lib = library("core")
    n = qkv.shape[0]
    write = k_pages is not None
    cols = (heads + (2 * kv_heads if write else 0)) * head_dim
    if qkv.shape[1] < cols:
        raise KernelError(f"qk_norm_rope_store: rows of {qkv.shape[1]} columns, {cols} needed")
    _f32vec(q_gain, head_dim, "q gain")
    _f32vec(k_gain, head_dim, "k gain")
    inv_freq = _rotary_table(inv_freq, rotary_dim)
    _i32(tok_req, "tok_req"), _i32(tok_pos, "tok_pos"), _i32(block_table, "block_table"), _i32(status, "status")
    page_size, n_pages = 1, 0
    if write:
        _check_pages(k_pages, v_pages, kv_heads, head_dim, qkv.dtype, "qk_norm_rope_store")
        page_size, n_pages = k_pages.shape[2], k_pages.shape[0]
    _launched(1)
    check(lib, lib.gb_qk_norm_rope_store(
        _ptr(qkv), dtype_code(qkv.dtype), _c_ll(_rows(qkv, "qkv")), _ptr(q_gain), _ptr(k_gain), _c_float(eps),
        _ptr(inv_freq), _c_int(rotary_dim), _c_int(1 if adjacent_pairs else 0), _ptr(tok_req), _ptr(tok_pos),
        _ptr(block_table), _c_int(block_table.shape[1] if block_table.dim() == 2 else 0), _c_int(page_size),
        _ptr(k_pages), _ptr(v_pages), _c_int(n_pages), _c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
        _c_int(1 if write else 0), _ptr(status), _stream()))


def qk_norm_rope_store_partials(qkv: Partials, q_out: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                                q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                                inv_freq: Optional[torch.Tensor], rotary_dim: int, adjacent_pairs: bool,
                                tok_req: torch.Tensor, tok_pos: torch.Tensor, block_table: torch.Tensor,
                                k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                                status: torch.Tensor) -> torch.Tensor:
    """As ``qk_norm_rope_store`` for q, k, v given as the partial tiles of their
    split-K product; q (normed and rotated) goes to ``q_out`` [n, heads*head_dim]."""
    _need_cuda(qkv.ws, qkv.bias, q_out, q_gain, k_gain, inv_freq, tok_req, tok_pos, block_table, k_pages, v_pages,
               status)
    lib = library("core")
    ws = qkv.ws
    n = ws.shape[1]
    write = k_pages is not None
    cols = (heads + (2 * kv_heads if write else 0)) * head_dim
    if ws.dtype != torch.float32 or not ws.is_contiguous() or ws.shape[2] != cols or qkv.dtype != torch.bfloat16:
        raise KernelError(f"qk_norm_rope_store_partials: partial tiles [splits, n, {cols}] float32 expected")
    if q_out.shape != (n, heads * head_dim) or q_out.dtype != torch.bfloat16 or not q_out.is_contiguous():
        raise KernelError("qk_norm_rope_store_partials: q_out must be contiguous bfloat16 [n, heads*head_dim]")
    _f32vec(qkv.bias, cols, "qkv bias")
    _f32vec(q_gain, head_dim, "q gain")
    _f32vec(k_gain, head_dim, "k gain")
    inv_freq = _rotary_table(inv_freq, rotary_dim)
    _i32(tok_req, "tok_req"), _i32(tok_pos, "tok_pos"), _i32(block_table, "block_table"), _i32(status, "status")
    page_size, n_pages = 1, 0
    if write:
        _check_pages(k_pages, v_pages, kv_heads, head_dim, torch.bfloat16, "qk_norm_rope_store_partials")
        page_size, n_pages = k_pages.shape[2], k_pages.shape[0]
    _launched(1)
    check(lib, lib.gb_qk_norm_rope_store_partials(
        _ptr(ws), _c_int(ws.shape[0]), _ptr(qkv.bias), _ptr(q_out), _ptr(q_gain), _ptr(k_gain), _c_float(eps),
        _ptr(inv_freq), _c_int(rotary_dim), _c_int(1 if adjacent_pairs else 0), _ptr(tok_req), _ptr(tok_pos),
        _ptr(block_table), _c_int(block_table.shape[1] if block_table.dim() == 2 else 0), _c_int(page_size),
        _ptr(k_pages), _ptr(v_pages), _c_int(n_pages), _c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
        _c_int(1 if write else 0), _ptr(status), _stream()))
    return q_out


def paged_attention(q: torch.Tensor, heads: int, kv_heads: int, head_dim: int, k_pages: torch.Tensor,
                    v_pages: torch.Tensor, block_table: torch.Tensor, tok_req: torch.Tensor, tok_pos: torch.Tensor,
                    scale: float, window: int, out: torch.Tensor, status: torch.Tensor, hints=None,
                    softcap: float = 0.0) -> torch.Tensor:
    """out[t, h, :] = softmax over visible keys of (q.K)*scale, times V; q may be
    a column slice of a wider row (its row stride is passed on).  ``hints`` is
    the step's state (per-request starts and lengths and the longest portion):
    with it, bfloat16 attention runs on the tensor cores.  ``softcap`` > 0: the
    scaled scores pass through cap * tanh(s / cap) (the generic kernel only)."""
    _need_cuda(q, k_pages, v_pages, block_table, tok_req, tok_pos, out, status)
    n = q.shape[0]
    if q.shape[1] != heads * head_dim or out.shape != (n, heads * head_dim) or q.dtype != out.dtype:
        raise KernelError("paged_attention: q and out must be [n, heads*head_dim] of one dtype")
    _check_pages(k_pages, v_pages, kv_heads, head_dim, q.dtype, "paged_attention")
    _i32(tok_req, "tok_req"), _i32(tok_pos, "tok_pos"), _i32(block_table, "block_table"), _i32(status, "status")
    if hints is not None and softcap <= 0 and q.dtype == torch.bfloat16 \
            and attention_tc_supported(q, out, heads, kv_heads, head_dim):
        return _attention_tc(q, heads, kv_heads, head_dim, k_pages, v_pages, block_table, scale, window, out,
                             status, hints)
    lib = library("core")
    _launched(1)
    check(lib, lib.gb_paged_attention(
        _ptr(q), dtype_code(q.dtype), _c_ll(_rows(q, "q")), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        _c_int(block_table.shape[1]), _c_int(k_pages.shape[2]), _c_int(k_pages.shape[0]), _ptr(tok_req),
        _ptr(tok_pos), _ptr(out), _c_ll(_rows(out, "out")), _c_int(n), _c_int(heads), _c_int(kv_heads),
        _c_int(head_dim), _c_float(scale), _c_float(softcap), _c_int(window or 0), _ptr(status), _stream()))
    return out


def scale_softcap(x: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """x <- x * scale, then cap * tanh(x / cap) when cap > 0, in place on contiguous float32."""
    _need_cuda(x)
    lib = library("core")
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_softcap: contiguous float32 values expected")
    _launched(1)
    check(lib, lib.gb_scale_softcap(_ptr(x), _c_ll(x.numel()), _c_float(scale), _c_float(cap), _stream()))
    return x


def attention_tc_supported(q, out, heads, kv_heads, head_dim) -> bool:
    return (head_dim % 16 == 0 and 16 <= head_dim <= 128 and heads % kv_heads == 0 and heads // kv_heads <= 64
            and q.stride(0) % 8 == 0 and out.stride(0) % 2 == 0 and q.data_ptr() % 16 == 0)


_ATTN_CTAS = int(os.environ.get("GIBBS_B200_ATTN_CTAS", "592"))   # about four CTAs per SM


def attention_splits(n_requests: int, kv_heads: int, max_ctx_len: int) -> int:
    """How many CTAs share the keys of one (request, kv head) when decoding:
    enough to occupy the GPU, at least two tiles of 64 keys each."""
    by_sm = max(1, _ATTN_CTAS // max(1, n_requests * kv_heads))      # about four CTAs per SM
    by_len = max(1, -(-max_ctx_len // 128))
    # up to 16 splits of at least two tiles; beyond that (up to the merge kernel's 32) only with 1,024 keys a split
    return max(1, min(by_sm, max(min(16, by_len), min(32, max_ctx_len // 1024))))


# prompt portions on tcgen05 (csrc/attention_tcgen05.cu); 0: keep them on the mma.sync kernel
_ATTN_TCGEN05 = os.environ.get("GIBBS_B200_ATTN_TCGEN05", "1") != "0"


def _attention_tc(q, heads, kv_heads, head_dim, k_pages, v_pages, block_table, scale, window, out, status, step):
    lib = library("tensorcore")
    n, group = q.shape[0], heads // kv_heads
    small = step.max_q_len * group <= 16 and group <= 16
    if not small and _ATTN_TCGEN05 and lib.gb_attention_tcgen05_supported(
            _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(k_pages.shape[2]), _c_ll(_rows(q, "q")),
            _c_ll(_rows(out, "out"))) and out.data_ptr() % 16 == 0 and scale > 0:
        rc = lib.gb_attention_tcgen05(
            _ptr(q), _c_ll(_rows(q, "q")), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
            _c_int(block_table.shape[1]), _c_int(k_pages.shape[2]), _c_int(k_pages.shape[0]), _ptr(step.q_start),
            _ptr(step.q_len), _ptr(step.start_pos), _ptr(out), _c_ll(_rows(out, "out")), _c_int(step.n_requests),
            _c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_float(scale), _c_int(window or 0),
            _ptr(status), _stream())
        if rc < 0:
            check(lib, rc)
        _launched(rc)
        return out
    splits = attention_splits(step.n_requests, kv_heads, step.max_ctx_len) if small else 1
    ws = None
    if splits > 1:
        ws = torch.empty(splits * n * heads * (head_dim + 2), dtype=torch.float32, device=q.device)
    rc = lib.gb_attention_tc(
        _ptr(q), _c_ll(_rows(q, "q")), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), _c_int(block_table.shape[1]),
        _c_int(k_pages.shape[2]), _c_int(k_pages.shape[0]), _ptr(step.q_start), _ptr(step.q_len),
        _ptr(step.start_pos), _ptr(out), _c_ll(_rows(out, "out")), _c_int(step.n_requests), _c_int(n),
        _c_int(step.max_q_len), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_float(scale),
        _c_int(window or 0), _c_int(splits), _ptr(ws), _ptr(status), _stream())
    if rc < 0:
        check(lib, rc)
    _launched(rc)
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           seed: Optional[torch.Tensor] = None, counter: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token id per logits row; per-row parameters (None: greedy)."""
    _need_cuda(logits, out, temperature, top_k, top_p, seed, counter)
    lib = library("core")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits are float32")
    _i32(out, "sample out"), _i32(top_k, "top_k")
    for t, w in ((temperature, "temperature"), (top_p, "top_p")):
        _f32vec(t, rows, "sample " + w)
    for t, w in ((seed, "seed"), (counter, "counter")):
        if t is not None and (t.dtype != torch.int64 or t.numel() != rows or not t.is_contiguous()):
            raise KernelError(f"sample {w}: expected {rows} int64 values")
    _launched(1)
    check(lib, lib.gb_sample(_ptr(logits), _c_ll(_rows(logits, "logits")), _c_int(rows), _c_int(vocab),
                             _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(counter), _ptr(out),
                             _stream()))
    return out


RECENT_TOKENS = 64          # how many of a request's latest tokens the repetition penalty looks at


def repetition_penalty(logits: torch.Tensor, recent: torch.Tensor, penalty: torch.Tensor,
                       temperature: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Applies the repetition penalty to ``logits`` [rows, vocab] in place: ``recent`` [rows, 64]
    int32 holds each row's latest token ids (-1 where there are fewer), ``penalty`` [rows] its
    factor (<= 1: the row is left alone), ``temperature`` [rows] selects the rule (None or
    <= 1e-4: the greedy one).  csrc/sampling.cu."""
    _need_cuda(logits, recent, penalty, temperature)
    lib = library("core")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("repetition_penalty: logits are float32")
    _i32(recent, "repetition_penalty recent")
    if recent.shape != (rows, RECENT_TOKENS) or not recent.is_contiguous():
        raise KernelError(f"repetition_penalty: recent must be contiguous int32 [{rows}, {RECENT_TOKENS}]")
    _f32vec(penalty, rows, "repetition_penalty penalty")
    _f32vec(temperature, rows, "repetition_penalty temperature")
    _launched(1)
    check(lib, lib.gb_repetition_penalty(_ptr(logits), _c_ll(_rows(logits, "logits")), _c_int(vocab), _ptr(recent),
                                         _ptr(penalty), _ptr(temperature), _c_int(rows), _stream()))
    return logits


def logprob_info(logits: torch.Tensor, chosen: torch.Tensor, k: int):
    """For each logits row: (probability of chosen[row], entropy of softmax(row), ids [rows, k] and
    probabilities [rows, k] of the k most probable tokens), all on the device."""
    _need_cuda(logits, chosen)
    lib = library("core")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("logprob_info: logits are float32")
    _i32(chosen, "logprob_info chosen")
    if chosen.numel() != rows:
        raise KernelError("logprob_info: one chosen id per row expected")
    dev = logits.device
    prob = torch.empty(rows, dtype=torch.float32, device=dev)
    entropy = torch.empty(rows, dtype=torch.float32, device=dev)
    ids = torch.empty((rows, k), dtype=torch.int32, device=dev)
    probs = torch.empty((rows, k), dtype=torch.float32, device=dev)
    _launched(1)
    check(lib, lib.gb_logprob_info(_ptr(logits), _c_ll(_rows(logits, "logits")), _c_int(rows), _c_int(vocab),
                                   _ptr(chosen), _c_int(k), _ptr(prob), _ptr(entropy), _ptr(ids), _ptr(probs),
                                   _stream()))
    return prob, entropy, ids, probs
