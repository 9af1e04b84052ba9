"""The entry point for callers that cannot allocate device memory
(``gb_linear_tc_no_alloc``, declared in ``gibbs_b200/csrc/gb_no_alloc.h``).

Such a caller (a plug-in without an allocator, code inside a stream capture, a
program that only has the C ABI) hands in inputs and an output and nothing
else; the kernel's split-K scratch is an array inside the library.  The test
therefore goes through the exported C symbol with raw pointers, never through
the Python wrappers, and compares with the ordinary entry point, which gets
its workspace from the caller.  It runs the call twice in a row, because the
second call finds the first call's leftovers in the shared scratch.

The file sorts last on purpose: if it fails, a run that stops at the first
failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 1 << 20


def _lib():
    from gibbs_b200.ops.library import library
    lib = library("tensorcore")
    lib.gb_linear_tc_no_alloc_needs.restype = ctypes.c_longlong
    lib.gb_last_error.restype = ctypes.c_char_p
    return lib


def _call(lib, a, w, bias, out, mode, status):
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)
    m, k = a.shape
    return lib.gb_linear_tc_no_alloc(
        p(a), ctypes.c_longlong(a.stride(0)), p(w), ctypes.c_longlong(w.stride(0)), p(bias), p(out), ctypes.c_int(mode),
        ctypes.c_longlong(out.stride(0)), ctypes.c_int(m), ctypes.c_int(w.shape[0]), ctypes.c_int(k), p(status),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _float64_product(a, w, bias, base, mode):
    """The same product restated in float64 (on the device, with the library's float64 matmul)."""
    y = a.double() @ w.double().T + bias.double()
    if mode == 3:                                   # gate and up rows alternate in blocks of 64
        y = y.reshape(y.shape[0], -1, 2, 64)
        g, u = y[:, :, 0, :].reshape(y.shape[0], -1), y[:, :, 1, :].reshape(y.shape[0], -1)
        return g / (1 + torch.exp(-g)) * u
    return y + base.double() if mode == 2 else y


# the last shape is one of more than 128 rows whose split (8 x 520 x 392 floats) would not fit the
# built-in scratch: it runs with K whole, and the ordinary entry point (which splits) is its witness
@pytest.mark.parametrize("m,n,k,mode", [(8, 2048, 2048, 2), (1, 3072, 2048, 0), (16, 2048, 8192, 1), (4, 256, 4096, 3),
                                        (300, 384, 520, 0), (520, 392, 4104, 1)])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(m, n, k, mode):
    from gibbs_b200 import ops
    lib = _lib()
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    n_out = n // 2 if mode == 3 else n
    out_dtype = torch.bfloat16 if mode in (0, 3) else torch.float32
    base = torch.randn(m, n_out, device=DEV).to(out_dtype)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    needs = lib.gb_linear_tc_no_alloc_needs(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
    assert needs <= MAX_FLOATS
    if m > 128:
        lib.gb_linear_tc_workspace.restype = ctypes.c_longlong
        would = lib.gb_linear_tc_workspace(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
        assert (needs == 0) == (would > MAX_FLOATS or would == 0)
    exact = _float64_product(a, w, bias, base, mode)
    for round_ in range(2):
        if round_ == 1:
            # another product in between leaves its own partial sums in the shared scratch
            other = torch.empty(2, 2048, dtype=torch.float32, device=DEV)
            assert _call(lib, a[:2].contiguous(), torch.ones(2048, k, device=DEV).to(torch.bfloat16), None, other, 1,
                         status) > 0
        want = base.clone()
        ops.linear_tc(a, w, bias, want, accumulate=(mode == 2), swiglu=(mode == 3))
        got = base.clone()
        rc = _call(lib, a, w, bias, got, mode, status)
        assert rc in (1, 2), lib.gb_last_error().decode()
        assert (rc == 2) == (needs > 0)
        torch.cuda.synchronize()
        # same kernels, same split, same order of addition: the tolerance of the kernel tests
        # (2e-2 relative for bfloat16 outputs, 2e-5 for 32-bit ones) is met with room to spare
        tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-5
        scale = want.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= tol * scale
        # and against the float64 restatement of the product itself
        assert (got.double() - exact).abs().max().item() <= tol * exact.abs().max().item()
        assert int(status.item()) == 0


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    m, n, k = 64, 6144, 2048                       # splits 3 ways: 1,179,648 floats of partial tiles
    a = torch.zeros(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(n, k, device=DEV, dtype=torch.bfloat16)
    out = torch.full((m, n), 7.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert lib.gb_linear_tc_no_alloc_needs(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k)) > MAX_FLOATS
    rc = _call(lib, a, w, None, out, 0, status)
    assert rc < 0
    msg = lib.gb_last_error().decode()
    assert "1179648" in msg and "1048576" in msg and "gb_linear_tc" in msg
    torch.cuda.synchronize()
    assert float(out.float().min()) == 7.0         # nothing was launched
    # a missing status word is refused too
    rc = lib.gb_linear_tc_no_alloc(ctypes.c_void_p(a.data_ptr()), ctypes.c_longlong(k), ctypes.c_void_p(w.data_ptr()),
                                   ctypes.c_longlong(k), ctypes.c_void_p(0), ctypes.c_void_p(out.data_ptr()),
                                   ctypes.c_int(0), ctypes.c_longlong(n), ctypes.c_int(1), ctypes.c_int(n),
                                   ctypes.c_int(k), ctypes.c_void_p(0), ctypes.c_void_p(0))
    assert rc < 0 and "status" in lib.gb_last_error().decode()
