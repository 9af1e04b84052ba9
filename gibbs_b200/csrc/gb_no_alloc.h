// gb_linear_tc_no_alloc: the bfloat16 tensor-core matrix product for callers
// that cannot allocate device memory.  MisterTK/gibbs has no counterpart of
// this entry point; it exists for this library's own users.
//
// Who needs it.  gb_linear_tc asks its caller for a 32-bit workspace whenever it
// splits K (small batches), so the caller must be able to allocate one.  Some
// callers cannot: code that runs while a stream is being captured into a graph
// (cudaMalloc is not allowed there), a plug-in inside a host application that
// owns all device memory and hands none out, a hard-real-time loop whose memory
// was fixed at start-up, or a program in another language that reaches this
// library through its C ABI and has no device allocator at hand.  For them the
// workspace is a fixed array that is part of this library's image on the GPU.
//
// What it costs and what it limits.
//  - The array holds GB_NO_ALLOC_MAX_WORKSPACE_FLOATS floats (4 MiB).  Every GPU
//    on which a process loads this library carries it until the process exits,
//    whether or not this function is ever called.
//  - A product of up to 128 rows whose split-K partial tiles (splits * M * N
//    floats, see gb_linear_tc_no_alloc_needs) do not fit is refused with
//    GB_ERR_ARG and a message that names the sizes; nothing is launched.
//    Products that do not split K need no scratch and are always taken.  Above
//    128 rows K is split for speed only: such a product whose partial tiles
//    would not fit runs with K whole instead (slower, same result up to the
//    order of the additions), and gb_linear_tc_no_alloc_needs says 0 for it.
//  - The function itself allocates nothing: no cudaMalloc, no cudaFree, no
//    library that allocates.  Inputs, the output and the status word are the
//    caller's.  The tensor maps it builds live on its stack.
//  - All calls on a device share the one array.  A call overwrites exactly the
//    part it will read back, so nothing needs clearing between calls and stale
//    contents of an earlier call are never read; but two calls that run on the
//    GPU at the same time (different streams, or two host threads) would write
//    the same floats and must not be issued.  Calls on one stream are safe.
//  - The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and keeps it.  Make that
//    first call outside any stream capture.
//  - W must be complete when the kernel starts.  The kernel asks for its first
//    weight tiles before it waits for the kernels ahead of it on the stream (it
//    is launched with programmatic stream serialization, so that a kernel
//    before it that signals griddepcontrol.launch_dependents lets it start
//    early).  After an ordinary kernel or copy this cannot matter; but if the
//    kernel right before it signals its dependents early AND writes W, put
//    something else between the two.  X, bias and out may come from that kernel.
//  - Launch limits (shared-memory size, SM count) are looked up once per process,
//    for the device that is current then: use it on GPUs of one kind.
//
// Arguments are those of gb_linear_tc without workspace and flags:
// X [M, K] bf16 (row stride ldx), W [N, K] bf16 (row stride ldw), bias f32 [N]
// or null; mode 0: out bf16 [M, N], 1: out f32, 2: out f32 +=, 3: SwiGLU over
// gate/up rows alternating in blocks of 64 (out bf16 [M, N / 2]); status: an
// int on the device that a kernel sets if a bounded wait runs out.  Returns the
// number of kernels launched (1 or 2) or a negative GbStatus; gb_last_error()
// has the message.
#pragma once
#include <cuda_runtime.h>

#define GB_NO_ALLOC_MAX_WORKSPACE_FLOATS (1 << 20)

extern "C" {
int gb_linear_tc_no_alloc(const void* X, long long ldx, const void* W, long long ldw, const float* bias, void* out,
                          int mode, long long ldo, int M, int N, int K, int* status, cudaStream_t stream);
// Floats of scratch the product would use (0 when K is not split); compare with
// GB_NO_ALLOC_MAX_WORKSPACE_FLOATS before calling.
long long gb_linear_tc_no_alloc_needs(int M, int N, int K);
}
