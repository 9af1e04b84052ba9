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
  float t = (threadIdx.x < nw) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

// NV sums over the `splits` partial tiles a split-K product left in 32-bit ([split][row][col],
// `stride` elements between splits), at the element offsets at[0..NV): the loads of four splits
// are requested together and the terms are added in split order.
template <int NV>
__device__ __forceinline__ void sum_partials(const float* __restrict__ ws, int splits, size_t stride,
                                             const size_t* at, float* acc) {
#pragma unroll
  for (int v = 0; v < NV; ++v) acc[v] = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 4) {
    float a[4][NV];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int v = 0; v < NV; ++v) a[u][v] = (s0 + u < splits) ? __ldcg(ws + (size_t)(s0 + u) * stride + at[v]) : 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u)
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
//     still touch (activations, caches, state; weights and launch arguments are
//     safe).  pdl_wait() returns when the earlier kernels have completed and
//     their writes are visible.
// Outside such a launch both are no-ops.  GIBBS_B200_PDL=0 turns the launch
// attribute off (kernels then run strictly one after the other).
//
// Pointers to anything an earlier kernel writes (activations, cache pages, state, a step's
// metadata) are NOT declared `const ... __restrict__`: the compiler takes loads through such a
// pointer for invariant and may move them above pdl_wait() (it did, in a kernel that fetched its
// first tile right after the wait).  Only what never changes while a model runs (weights, gains,
// taps, biases, tables) keeps the qualifier.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

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
