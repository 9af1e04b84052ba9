// Shared helpers of the gibbs_b200 kernels: element types, 32-bit conversion,
// warp reductions and the C-ABI error convention.
//
// Every exported function returns 0 on success and a negative code otherwise;
// gb_last_error() gives the message of the last failure on the calling thread.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define GB_API extern "C" __attribute__((visibility("default")))

enum GbDtype : int { GB_F32 = 0, GB_BF16 = 1 };

enum GbStatus : int {
  GB_OK = 0,
  GB_ERR_ARG = -1,      // a size or option the kernel does not take
  GB_ERR_CUDA = -2,     // the launch failed
  GB_ERR_TIMEOUT = -3,  // a bounded device-side wait ran out
};

char* gb_error_buffer();  // thread-local, 512 bytes (defined in errors.cu)

#define GB_FAIL(code, ...)                              \
  do {                                                  \
    snprintf(gb_error_buffer(), 512, __VA_ARGS__);      \
    return (code);                                      \
  } while (0)

#define GB_CHECK_LAUNCH(name)                                                        \
  do {                                                                               \
    cudaError_t e_ = cudaGetLastError();                                             \
    if (e_ != cudaSuccess) GB_FAIL(GB_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e_)); \
  } while (0)

#define GB_CUDA(call)                                                                \
  do {                                                                               \
    cudaError_t e_ = (call);                                                         \
    if (e_ != cudaSuccess) GB_FAIL(GB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  const float t = (lane < nw) ? scratch[lane] : 0.f;
  return warp_sum(t);            // every warp adds the same values in the same order
}

// Asynchronous 16-byte copies from global (through L2) to shared memory: every copy a thread issues
// is in flight at once, whatever the compiler makes of the code around it, and holds no register.
// A thread that reads only what it copied itself needs gb_cp_async_wait_all() and no barrier.
__device__ __forceinline__ void gb_cp_async_16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
               ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void gb_cp_async_4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;"
               ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void gb_cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// L2 loads that are issued where they stand (the compiler neither sinks them to their first use
// nor drops them, and keeps them behind pdl_wait(), which is a volatile asm too): a batch of them
// written one after the other is in flight together.  Use these, not __ldcg, for 16-bit types:
// the header's __ldcg of a bfloat16 is a plain asm without a memory operand, which the compiler
// treats as a function of the pointer's value and may move above the wait or out of a loop.
__device__ __forceinline__ float ldcg_now(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ bf16 ldcg_now(const bf16* p) {
  unsigned short v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return __ushort_as_bfloat16(v);
}
__device__ __forceinline__ float4 ldcg_now(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// NV sums over the `splits` partial tiles a split-K product left in 32-bit ([split][row][col],
// `stride` elements between splits), at the element offsets at[0..NV): the loads of eight splits
// are requested together (one trip to L2) and the terms are added in split order.
template <int NV>
__device__ __forceinline__ void sum_partials(const float* ws, int splits, size_t stride,
                                             const size_t* at, float* acc) {
#pragma unroll
  for (int v = 0; v < NV; ++v) acc[v] = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 8) {
    float a[8][NV];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      // (a split past the last one re-reads the last one and is not added: no branch around a load)
      const int su = s0 + u < splits ? s0 + u : splits - 1;
#pragma unroll
      for (int v = 0; v < NV; ++v) a[u][v] = ldcg_now(ws + (size_t)su * stride + at[v]);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (s0 + u < splits) {
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v] += a[u][v];
      }
  }
}

static inline int gb_div_up(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---------------------------------------------------------------- launches
// Programmatic dependent launch: a kernel launched through gb_launch may begin
// (become resident, run its prologue) while the kernel before it on the stream
// is still running.  Every kernel of this library therefore
//   - calls pdl_trigger() first, which lets the kernel after it start early, and
//   - calls pdl_wait() before it reads or writes anything an earlier kernel may
//     still touch (activations, caches, state).  pdl_wait() returns when the
//     earlier kernels have completed and their writes are visible.
// Outside such a launch both are no-ops.  GIBBS_B200_PDL=0 turns the launch
// attribute off (kernels then run strictly one after the other).
//
// What may be read BEFORE pdl_wait(), so that its trip to L2 is over when the wait returns:
//   - weights, gains, taps, biases, tables and launch arguments: nothing writes them while a model runs;
//   - a step's metadata (token->request, positions, lengths, slot ids, block tables, row lists): a
//     host copy writes it, and that copy completes before the step's first kernel starts.  The one
//     exception are the token ids, which feed_tokens_kernel may rewrite: only the embedding gather
//     reads them, after its wait;
//   - cache pages and state at positions that earlier STEPS wrote (not this step's own tokens).
//
// Pointers to anything an earlier kernel writes (activations, cache pages, state) are NOT declared
// `const ... __restrict__`: the compiler takes loads through such a pointer for invariant and may
// move them above pdl_wait() (it did, in a kernel that fetched its first tile right after the
// wait).  Only what never changes while a model runs keeps the qualifier.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// gb_pin(v): what was computed or loaded into v stays where the program wrote it.  The loads a
// kernel issues before pdl_wait() come from `const __restrict__` pointers, which the compiler may
// sink to their first use, i.e. behind the wait, where each of them becomes a trip to L2 on the
// step's critical path again (measured: 2.9 against 6.0 us for the same kernel).  An empty volatile
// asm that takes the value as an operand keeps its computation in front of the next volatile asm,
// which pdl_wait() is; it emits no instruction and waits for nothing.
__device__ __forceinline__ void gb_pin(float& v) { asm volatile("" : "+f"(v)); }
__device__ __forceinline__ void gb_pin(int& v) { asm volatile("" : "+r"(v)); }
__device__ __forceinline__ void gb_pin(long long& v) { asm volatile("" : "+l"(v)); }
__device__ __forceinline__ void gb_pin(bool& v) {
  int t = v;
  asm volatile("" : "+r"(t));
  v = t != 0;
}
__device__ __forceinline__ void gb_pin(float4& v) { asm volatile("" : "+f"(v.x), "+f"(v.y), "+f"(v.z), "+f"(v.w)); }
template <typename T>
__device__ __forceinline__ void gb_pin(T*& p) {
  unsigned long long a = reinterpret_cast<unsigned long long>(p);
  asm volatile("" : "+l"(a));
  p = reinterpret_cast<T*>(a);
}

int gb_pdl_enabled();  // defined in errors.cu (one copy per shared library)

template <typename... KArgs, typename... Args>
inline cudaError_t gb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = gb_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
