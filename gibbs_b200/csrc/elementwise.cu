// Row-wise kernels that are bound by memory traffic: embedding gather,
// RMSNorm (with an optional row gather), SwiGLU over a fused [gate | up] row.
//
// Formulas (MisterTK/gibbs): embedding src/graph/cpu.rs:161-248; RMSNorm
// src/model/simd.rs:73-111 (scale = 1/sqrt(sum/n + eps), out = x*scale*g);
// SwiGLU src/graph/cpu.rs:378-390 ((g*sigmoid(g))*u).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* ids, float* __restrict__ out,
                             int dim, int vocab) {
  pdl_trigger();
  const int row = blockIdx.x;
  pdl_wait();
  int id = __ldcg(ids + row);                              // (through L2: the kernel in front may have rewritten it)
  // Token ids are checked on the host before the step; a bad id reads row 0.
  if (id < 0 || id >= vocab) id = 0;
  const T* src = table + (size_t)id * dim;
  float* dst = out + (size_t)row * dim;
  if (sizeof(T) == 2 && dim % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
    // a bfloat16 row in 16-byte pieces: each thread's loads are requested before any is used
    const uint4* s8 = reinterpret_cast<const uint4*>(src);
    const int n8 = dim >> 3;
    for (int c0 = threadIdx.x; c0 < n8; c0 += 4 * blockDim.x) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x;
        raw[u] = s8[c < n8 ? c : c0];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x;
        if (c < n8) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
          const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
          const float2 e = __bfloat1622float2(h[2]), f = __bfloat1622float2(h[3]);
          reinterpret_cast<float4*>(dst)[2 * c] = make_float4(a.x, a.y, b.x, b.y);
          reinterpret_cast<float4*>(dst)[2 * c + 1] = make_float4(e.x, e.y, f.x, f.y);
        }
      }
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x)
      dst[d] = to_f32(src[d]);
  }
}

GB_API int gb_embed(const void* table, int table_dtype, const int* ids, float* out, int n, int dim, int vocab,
                    cudaStream_t stream) {
  if (n <= 0) return GB_OK;
  const int threads = dim >= 1024 ? 256 : 128;
  if (table_dtype == GB_F32)
    gb_launch(embed_kernel<float>, dim3(n), dim3(threads), 0, stream, (const float*)table, ids, out, dim, vocab);
  else if (table_dtype == GB_BF16)
    gb_launch(embed_kernel<bf16>, dim3(n), dim3(threads), 0, stream, (const bf16*)table, ids, out, dim, vocab);
  else
    GB_FAIL(GB_ERR_ARG, "gb_embed: unknown table dtype %d", table_dtype);
  GB_CHECK_LAUNCH("gb_embed");
  return GB_OK;
}

// ---------------------------------------------------------------- token feedback
// ids[t] = picked[from[t]] where from[t] >= 0: the tokens a step's sampler picked feed the
// next step's gather without a trip through the host (the reference's Metal stream does
// the same with the id its argmax head wrote, src/backend/metal/program.rs:458-544).
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* picked,
                                   const int* from, int n, int n_picked) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int f = from[t];
  if (f >= 0 && f < n_picked) ids[t] = picked[f];
}

GB_API int gb_feed_tokens(int* ids, const int* picked, const int* from, int n, int n_picked, cudaStream_t stream) {
  if (n <= 0) return GB_OK;
  gb_launch(feed_tokens_kernel, dim3(gb_div_up(n, 128)), dim3(128), 0, stream, ids, picked, from, n, n_picked);
  GB_CHECK_LAUNCH("gb_feed_tokens");
  return GB_OK;
}

// ---------------------------------------------------------------- RMSNorm
// One block per output row.  `rows` (optional) gathers input rows.  The sum of
// squares is taken in a fixed order, so a row's result does not depend on
// what else is in the batch.
//
// `pend` (optional): partial sums [splits][n_src_rows][dim] (+ pend_bias) that a
// split-K product left to be added to x.  They are added here, in split order,
// before the statistics; without a row gather the sum is also written back to x
// (the residual stream carries on from it).
template <typename TOut>
__device__ __forceinline__ void store4(TOut* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = u;
}

// VEC > 0: dim is a multiple of 4, rows are 16-byte aligned and each thread keeps its
// VEC float4 of the row in registers (all loads of the row and of the partial sums are
// issued together; the row is read once).  VEC == 0: any dim, two passes.
// PEND: how many splits' loads are requested together (0: the kernel takes no partial sums).
// Instantiated apart so that rows without partial sums, or with one tile set (prompts), do not
// pay for the registers that hold eight splits' worth of loads.
template <typename TOut, int VEC, int PEND>
__device__ __forceinline__ void rmsnorm_body(float* __restrict__ x, long long ldx, const float* __restrict__ gain,
                                             TOut* __restrict__ out, const int* rows, int dim, float eps,
                                             const float* pend, int splits, long long n_src_rows,
                                             const float* __restrict__ pend_bias) {
  __shared__ float scratch[32];
  pdl_trigger();
  // What no kernel of the step writes (the gain, the row list from the step's metadata) is read
  // before the wait for the kernel in front: one trip to L2 less after it.
  const int r = blockIdx.x;
  long long sr = rows ? rows[r] : r;
  gb_pin(sr);
  float4 g4[VEC > 0 ? VEC : 1];
  if (VEC > 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      g4[i] = c < (dim >> 2) ? reinterpret_cast<const float4*>(gain)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
      gb_pin(g4[i]);
    }
  }
  float* src = x + (size_t)sr * ldx;
  TOut* dst = out + (size_t)r * dim;
  if constexpr (VEC > 0) {
  pdl_wait();
  const bool write_back = pend != nullptr && rows == nullptr;
  float ss = 0.f;
  float4 v[VEC > 0 ? VEC : 1];
  const int n4 = dim >> 2;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < n4 ? __ldcg(reinterpret_cast<const float4*>(src) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (PEND > 0 && pend) {
    // the partial sums of up to PEND splits are requested together (one trip to L2, not one
    // per split) and then added in split order
    constexpr int G = PEND > 0 ? PEND : 1;
    const size_t split_stride = (size_t)n_src_rows * dim;
    const float* p0 = pend + (size_t)sr * dim;
    for (int s0 = 0; s0 < splits; s0 += G) {
      float4 a[G][VEC > 0 ? VEC : 1];
#pragma unroll
      for (int u = 0; u < G; ++u) {
        // (a split past the last one re-reads the last one and is not added: loads without a
        // branch around them all go out together)
        const int su = s0 + u < splits ? s0 + u : splits - 1;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int c = threadIdx.x + i * blockDim.x;
          a[u][i] = ldcg_now(reinterpret_cast<const float4*>(p0 + (size_t)su * split_stride) + (c < n4 ? c : 0));
        }
      }
#pragma unroll
      for (int u = 0; u < G; ++u) {
        if (s0 + u < splits) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < n4) { v[i].x += a[u][i].x; v[i].y += a[u][i].y; v[i].z += a[u][i].z; v[i].w += a[u][i].w; }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < n4) {
        if (pend_bias) {
          const float4 b = reinterpret_cast<const float4*>(pend_bias)[c];
          v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
        }
        if (write_back) reinterpret_cast<float4*>(src)[c] = v[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < n4) {
      const float4 g = g4[i];
      store4<TOut>(dst + 4 * c, make_float4(v[i].x * scale * g.x, v[i].y * scale * g.y, v[i].z * scale * g.z,
                                            v[i].w * scale * g.w));
    }
  }
    return;
  } else {
  pdl_wait();
  const bool write_back = pend != nullptr && rows == nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float v = src[d];
    if (pend) {
      for (int s = 0; s < splits; ++s) v += pend[((size_t)s * n_src_rows + sr) * dim + d];
      if (pend_bias) v += pend_bias[d];
      if (write_back) src[d] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float v = src[d];                       // each thread re-reads what it wrote itself
    if (pend && !write_back) {
      for (int s = 0; s < splits; ++s) v += pend[((size_t)s * n_src_rows + sr) * dim + d];
      if (pend_bias) v += pend_bias[d];
    }
    dst[d] = from_f32<TOut>(v * scale * gain[d]);
  }
  }
}

// Rows to which a split-K product's partial sums are still to be added (decode steps): every
// thread copies its 16-byte pieces of all splits to shared memory asynchronously, so that all of
// them are one trip to L2, and then adds them in split order.  dim % 4 == 0; shared memory:
// splits * dim floats.
template <typename TOut>
__global__ void __launch_bounds__(1024) rmsnorm_splits_kernel(float* x, long long ldx, const float* __restrict__ gain,
                                                              TOut* __restrict__ out, const int* rows, int dim,
                                                              float eps, const float* pend, int splits,
                                                              long long n_src_rows,
                                                              const float* __restrict__ pend_bias) {
  extern __shared__ __align__(16) float parts[];            // [splits][dim]
  __shared__ float scratch[32];
  pdl_trigger();
  const int r = blockIdx.x;
  long long sr = rows ? rows[r] : r;
  gb_pin(sr);
  const int n4 = dim >> 2;
  constexpr int MAXV = 2;                                    // pieces per thread (the launch sees to it)
  float4 g4[MAXV], b4[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    g4[i] = c < n4 ? reinterpret_cast<const float4*>(gain)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    b4[i] = (pend_bias && c < n4) ? reinterpret_cast<const float4*>(pend_bias)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    gb_pin(g4[i]);
    gb_pin(b4[i]);
  }
  float* src = x + (size_t)sr * ldx;
  const float* p0 = pend + (size_t)sr * dim;
  long long split_stride = n_src_rows * dim;
  TOut* dst = out + (size_t)r * dim;
  gb_pin(src);                                               // (addresses too are ready before the wait)
  gb_pin(p0);
  gb_pin(split_stride);
  gb_pin(dst);
  pdl_wait();
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < n4)
      for (int s = 0; s < splits; ++s) gb_cp_async_16(parts + (size_t)s * dim + 4 * c, p0 + (size_t)s * split_stride + 4 * c);
  }
  float4 v[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < n4 ? ldcg_now(reinterpret_cast<const float4*>(src) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  gb_cp_async_wait_all();
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < n4) {
      for (int s = 0; s < splits; ++s) {
        const float4 a = *reinterpret_cast<const float4*>(parts + (size_t)s * dim + 4 * c);
        v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
      }
      if (pend_bias) { v[i].x += b4[i].x; v[i].y += b4[i].y; v[i].z += b4[i].z; v[i].w += b4[i].w; }
      if (rows == nullptr) reinterpret_cast<float4*>(src)[c] = v[i];
    }
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < n4)
      store4<TOut>(dst + 4 * c, make_float4(v[i].x * scale * g4[i].x, v[i].y * scale * g4[i].y,
                                            v[i].z * scale * g4[i].z, v[i].w * scale * g4[i].w));
  }
}

// MAXT: the most threads a launch of this variant uses (it bounds the registers a thread may take;
// the variants that keep many splits' loads in flight need more than a 1,024-thread block leaves).
template <typename TOut, int VEC, int PEND, int MAXT>
__global__ void __launch_bounds__(MAXT) rmsnorm_kernel(float* x, long long ldx, const float* gain, TOut* out,
                                                       const int* rows, int dim, float eps, const float* pend,
                                                       int splits, long long n_src_rows, const float* pend_bias) {
  rmsnorm_body<TOut, VEC, PEND>(x, ldx, gain, out, rows, dim, eps, pend, splits, n_src_rows, pend_bias);
}

template <typename TOut>
void launch_rmsnorm(float* x, long long ldx, const float* gain, TOut* out, const int* rows, int n_rows, int dim,
                    float eps, const float* pend, int splits, long long n_src_rows, const float* pend_bias,
                    cudaStream_t stream) {
  const bool vec_ok = dim % 4 == 0 && ldx % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)gain & 15) == 0 &&
                      ((uintptr_t)out & 15) == 0 && ((uintptr_t)pend & 15) == 0 && ((uintptr_t)pend_bias & 15) == 0;
  const int n4 = dim / 4;
  if (vec_ok && n4 <= 2 * 1024) {
    int threads = 32;
    while (threads < 1024 && threads < n4) threads <<= 1;
    const int g = pend ? (splits > 1 ? 8 : 1) : 0;
#define GB_NORM_LAUNCH(VEC, PEND, MAXT, THREADS)                                                                       \
    gb_launch(rmsnorm_kernel<TOut, VEC, PEND, MAXT>, dim3(n_rows), dim3(THREADS), 0, stream, x, ldx, gain, out, rows,  \
              dim, eps, pend, splits, n_src_rows, pend_bias)
    if (g == 8) {
      // Several splits to add: through shared memory while the splits fit there, else two pieces
      // per thread with the loads of four splits at a time in registers.
      const size_t smem = (size_t)splits * dim * sizeof(float);
      if (smem <= 160 * 1024) {
        static bool attr_set = false;
        if (!attr_set) {
          cudaFuncSetAttribute(rmsnorm_splits_kernel<TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
          attr_set = true;
        }
        int th = 32;
        while (th < 1024 && 2 * th < n4) th <<= 1;      // one piece per thread up to 1,024 columns... two above
        if (th < n4 && th < 1024) th <<= 1;
        gb_launch(rmsnorm_splits_kernel<TOut>, dim3(n_rows), dim3(th), smem, stream, x, ldx, gain, out, rows, dim, eps,
                  pend, splits, n_src_rows, pend_bias);
      } else {
        GB_NORM_LAUNCH(2, 4, 1024, 1024);
      }
      return;
    }
    if (threads > 256 && n4 <= 2 * 256) threads = 256;
    if (n4 <= threads) {
      if (g == 1) GB_NORM_LAUNCH(1, 1, 1024, threads);
      else GB_NORM_LAUNCH(1, 0, 1024, threads);
    } else if (threads <= 256) {
      if (g == 1) GB_NORM_LAUNCH(2, 1, 256, threads);
      else GB_NORM_LAUNCH(2, 0, 256, threads);
    } else {
      if (g == 1) GB_NORM_LAUNCH(2, 1, 1024, threads);
      else GB_NORM_LAUNCH(2, 0, 1024, threads);
    }
    return;
  }
  int threads = 32;
  while (threads < 512 && threads * 4 < dim) threads <<= 1;
  GB_NORM_LAUNCH(0, 8, 1024, threads);
#undef GB_NORM_LAUNCH
}

GB_API int gb_rmsnorm(float* x, long long ldx, const float* gain, void* out, int out_dtype, const int* rows,
                      int n_rows, int dim, float eps, const float* pend, int splits, long long n_src_rows,
                      const float* pend_bias, cudaStream_t stream) {
  if (n_rows <= 0) return GB_OK;
  if (out_dtype == GB_F32)
    launch_rmsnorm<float>(x, ldx, gain, (float*)out, rows, n_rows, dim, eps, pend, splits, n_src_rows, pend_bias,
                          stream);
  else if (out_dtype == GB_BF16)
    launch_rmsnorm<bf16>(x, ldx, gain, (bf16*)out, rows, n_rows, dim, eps, pend, splits, n_src_rows, pend_bias,
                         stream);
  else
    GB_FAIL(GB_ERR_ARG, "gb_rmsnorm: unknown output dtype %d", out_dtype);
  GB_CHECK_LAUNCH("gb_rmsnorm");
  return GB_OK;
}

// x[m, :] += sum over splits of pend[s][m, :] (+ bias), in split order.
__global__ void add_pending_kernel(float* __restrict__ x, long long ldx, const float* pend, int splits,
                                   const float* __restrict__ bias, long long n_rows, int dim) {
  pdl_trigger();
  pdl_wait();
  const long long total = n_rows * dim;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / dim;
    const int d = (int)(i - m * dim);
    float v = x[(size_t)m * ldx + d];
    for (int s = 0; s < splits; ++s) v += pend[(size_t)s * total + i];
    if (bias) v += bias[d];
    x[(size_t)m * ldx + d] = v;
  }
}

GB_API int gb_add_pending(float* x, long long ldx, const float* pend, int splits, const float* bias,
                          long long n_rows, int dim, cudaStream_t stream) {
  const long long total = n_rows * dim;
  if (total <= 0 || splits <= 0) return GB_OK;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  gb_launch(add_pending_kernel, dim3(blocks), dim3(256), 0, stream, x, ldx, pend, splits, bias, n_rows, dim);
  GB_CHECK_LAUNCH("gb_add_pending");
  return GB_OK;
}

// ---------------------------------------------------------------- SwiGLU
// in: [n, 2*inner] rows of [gate | up]; out: [n, inner].
template <typename T>
__global__ void swiglu_kernel(const T* gu, T* __restrict__ out, long long total, int inner) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / inner;
    const int c = (int)(i - row * inner);
    const float g = to_f32(gu[row * 2 * inner + c]);
    const float u = to_f32(gu[row * 2 * inner + inner + c]);
    const float sig = 1.0f / (1.0f + expf(-g));
    out[i] = from_f32<T>((g * sig) * u);
  }
}

GB_API int gb_swiglu(const void* gu, void* out, int dtype, int n, int inner, cudaStream_t stream) {
  const long long total = (long long)n * inner;
  if (total <= 0) return GB_OK;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == GB_F32)
    gb_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out, total, inner);
  else if (dtype == GB_BF16)
    gb_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out, total, inner);
  else
    GB_FAIL(GB_ERR_ARG, "gb_swiglu: unknown dtype %d", dtype);
  GB_CHECK_LAUNCH("gb_swiglu");
  return GB_OK;
}

// ---------------------------------------------------------------- logits: scale and soft cap
// x <- x * scale, then (cap > 0) x <- cap * tanh(x / cap), in place on 32-bit logits
// (MisterTK/gibbs arch/lib/transformer.json5:170-175: divided by logit_scale, then soft-capped).
__global__ void scale_softcap_kernel(float* x, long long total, float scale, float cap) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    x[i] = v;
  }
}

GB_API int gb_scale_softcap(float* x, long long total, float scale, float cap, cudaStream_t stream) {
  if (total <= 0) return GB_OK;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  gb_launch(scale_softcap_kernel, dim3(blocks), dim3(threads), 0, stream, x, total, scale, cap);
  GB_CHECK_LAUNCH("gb_scale_softcap");
  return GB_OK;
}

// ---------------------------------------------------------------- cast
template <typename TIn, typename TOut>
__global__ void cast_kernel(const TIn* in, TOut* __restrict__ out, long long total) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<TOut>(to_f32(in[i]));
}

GB_API int gb_cast(const void* in, int in_dtype, void* out, int out_dtype, long long total, cudaStream_t stream) {
  if (total <= 0) return GB_OK;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (in_dtype == GB_F32 && out_dtype == GB_BF16)
    gb_launch(cast_kernel<float, bf16>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, (bf16*)out, total);
  else if (in_dtype == GB_BF16 && out_dtype == GB_F32)
    gb_launch(cast_kernel<bf16, float>, dim3(blocks), dim3(threads), 0, stream, (const bf16*)in, (float*)out, total);
  else
    GB_FAIL(GB_ERR_ARG, "gb_cast: unsupported conversion %d -> %d", in_dtype, out_dtype);
  GB_CHECK_LAUNCH("gb_cast");
  return GB_OK;
}
