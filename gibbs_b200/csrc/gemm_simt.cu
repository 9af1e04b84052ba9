// out[m, n] (+)= sum_k A[m, k] * W[n, k] (+ bias[n]) with 32-bit FMA on the CUDA
// cores: the matrix product of the true 32-bit path, and of any operand pair
// the tensor-core kernel does not take (a weight kept in 32-bit beside 16-bit
// activations, sizes it refuses).  No tensor-core mode of any kind is used.
//
// Each output element is one accumulator that walks k in ascending order, so
// its value does not depend on the tile shape or on the rows beside it: the
// three kernels below (a general one, one with 128 x 128 tiles and 8 x 8
// outputs per thread for prompts, one with 16-column tiles for a few rows
// that spreads a narrow weight over many blocks) give the same bits.
// (MisterTK/gibbs Linear: src/graph/cpu.rs:249-274, 2338-2417; its blocked
// 32-bit product: src/model/nn.rs:383-529.)
#include "common.cuh"

namespace {

// Four consecutive elements of a row as 32-bit values (rows are 16-byte / 8-byte aligned).  The
// loads go through L2 (ld.global.cg), never through the read-only path: the activations were
// written by the kernel before this one, and a load the compiler takes for invariant may be moved
// above the wait for that kernel (it was, with the first k-block fetched right after the wait).
__device__ __forceinline__ float4 load4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 u = __ldcg(reinterpret_cast<const uint2*>(p));
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

__device__ __forceinline__ void store_out(void* out, int out_dtype, int accumulate, size_t o, float v) {
  if (out_dtype == GB_F32) {
    float* of = (float*)out;
    of[o] = accumulate ? of[o] + v : v;
  } else {
    ((bf16*)out)[o] = __float2bfloat16_rn(v);
  }
}

// ---- prompts: 128 x 128 tiles, 256 threads, 8 x 8 outputs per thread, k-blocks of 16 fetched into
// registers while the block before is multiplied.  K and the row strides are multiples of 4.
constexpr int LT = 128;     // tile edge
constexpr int LK = 16;
constexpr int LPAD = 4;

template <typename TA, typename TW>
__global__ void __launch_bounds__(256, 2)
gemm_simt_tile128_kernel(const TA* A, long long lda, const TW* __restrict__ W, long long ldw,
                         const float* __restrict__ bias, void* __restrict__ out, long long ldo, int out_dtype,
                         int accumulate, int M, int N, int K) {
  pdl_trigger();
  pdl_wait();
  __shared__ __align__(16) float As[LK][LT + LPAD];
  __shared__ __align__(16) float Ws[LK][LT + LPAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * LT, n0 = blockIdx.x * LT;
  // what this thread fetches of a k-block: 4 consecutive k of rows lr and lr + 64 of both tiles
  const int lr = tid >> 2, lk = (tid & 3) * 4;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float4 fa[2], fw[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gm = m0 + lr + 64 * h, gn = n0 + lr + 64 * h, gk = k0 + lk;
      fa[h] = (gm < M && gk < K) ? load4(A + (size_t)gm * lda + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
      fw[h] = (gn < N && gk < K) ? load4(W + (size_t)gn * ldw + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = lr + 64 * h;
      As[lk][r] = fa[h].x; As[lk + 1][r] = fa[h].y; As[lk + 2][r] = fa[h].z; As[lk + 3][r] = fa[h].w;
      Ws[lk][r] = fw[h].x; Ws[lk + 1][r] = fw[h].y; Ws[lk + 2][r] = fw[h].z; Ws[lk + 3][r] = fw[h].w;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += LK) {
    stash();
    __syncthreads();
    if (k0 + LK < K) fetch(k0 + LK);
#pragma unroll
    for (int k = 0; k < LK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[k][64 + ty * 4]);
      const float4 w0 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float4 w1 = *reinterpret_cast<const float4*>(&Ws[k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      store_out(out, out_dtype, accumulate, (size_t)gm * ldo + gn, v);
    }
  }
}

// ---- a few rows (decode): a block takes 16 columns of the weight and up to 16 rows, one output per
// thread, k-blocks of 64 fetched into registers while the block before is multiplied.  A weight of
// N rows is spread over N / 16 blocks, so that also a narrow weight is streamed by the whole GPU.
constexpr int SK = 64;

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_simt_rows16_kernel(const TA* A, long long lda, const TW* __restrict__ W, long long ldw,
                        const float* __restrict__ bias, void* __restrict__ out, long long ldo, int out_dtype,
                        int accumulate, int M, int N, int K) {
  pdl_trigger();
  pdl_wait();
  __shared__ float As[16][SK + 1];
  __shared__ float Ws[16][SK + 1];
  const int tid = threadIdx.x;
  const int tn = tid & 15, tm = tid >> 4;            // this thread's output: row tm, column n0 + tn
  const int n0 = blockIdx.x * 16;
  const int lr = tid >> 4, lk = (tid & 15) * 4;       // what it fetches: 4 consecutive k of row lr of both tiles
  float acc = 0.f;
  float4 fa, fw;
  auto fetch = [&](int k0) {
    const int gk = k0 + lk;
    fa = (lr < M && gk < K) ? load4(A + (size_t)lr * lda + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
    fw = (n0 + lr < N && gk < K) ? load4(W + (size_t)(n0 + lr) * ldw + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += SK) {
    As[lr][lk] = fa.x; As[lr][lk + 1] = fa.y; As[lr][lk + 2] = fa.z; As[lr][lk + 3] = fa.w;
    Ws[lr][lk] = fw.x; Ws[lr][lk + 1] = fw.y; Ws[lr][lk + 2] = fw.z; Ws[lr][lk + 3] = fw.w;
    __syncthreads();
    if (k0 + SK < K) fetch(k0 + SK);
#pragma unroll
    for (int k = 0; k < SK; ++k) acc = fmaf(As[tm][k], Ws[tn][k], acc);
    __syncthreads();
  }
  const int gn = n0 + tn;
  if (tm < M && gn < N) {
    float v = acc;
    if (bias) v += bias[gn];
    store_out(out, out_dtype, accumulate, (size_t)tm * ldo + gn, v);
  }
}

// ---- the general kernel: any sizes and strides

constexpr int BN = 64;
constexpr int BK = 16;

template <typename TA, typename TW, int TM>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* A, long long lda, const TW* __restrict__ W, long long ldw,
                 const float* __restrict__ bias, void* __restrict__ out, long long ldo, int out_dtype,
                 int accumulate, int M, int N, int K) {
  pdl_trigger();
  pdl_wait();
  constexpr int BM = 16 * TM;
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += 256) {
      const int m = idx / BK, k = idx % BK;
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
    }
    for (int idx = tid; idx < BN * BK; idx += 256) {
      const int n = idx / BK, k = idx % BK;
      const int gn = n0 + n, gk = k0 + k;
      Ws[k][n] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], w[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      store_out(out, out_dtype, accumulate, (size_t)gm * ldo + gn, v);
    }
  }
}

template <typename TA, typename TW>
void launch(const void* A, long long lda, const void* W, long long ldw, const float* bias, void* out, long long ldo,
            int out_dtype, int accumulate, int M, int N, int K, cudaStream_t stream) {
  const bool rows4 = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && ((uintptr_t)A % (4 * sizeof(TA))) == 0 &&
                     ((uintptr_t)W % (4 * sizeof(TW))) == 0;
  if (rows4 && M <= 16) {
    gb_launch(gemm_simt_rows16_kernel<TA, TW>, dim3(gb_div_up(N, 16)), dim3(256), 0, stream, (const TA*)A, lda,
              (const TW*)W, ldw, bias, out, ldo, out_dtype, accumulate, M, N, K);
  } else if (rows4 && M > 64) {
    dim3 grid(gb_div_up(N, LT), gb_div_up(M, LT));
    gb_launch(gemm_simt_tile128_kernel<TA, TW>, dim3(grid), dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W,
              ldw, bias, out, ldo, out_dtype, accumulate, M, N, K);
  } else if (M <= 16) {
    dim3 grid(gb_div_up(N, BN), gb_div_up(M, 16));
    gb_launch(gemm_simt_kernel<TA, TW, 1>, dim3(grid), dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, bias, out, ldo,
                                                          out_dtype, accumulate, M, N, K);
  } else {
    dim3 grid(gb_div_up(N, BN), gb_div_up(M, 64));
    gb_launch(gemm_simt_kernel<TA, TW, 4>, dim3(grid), dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, bias, out, ldo,
                                                          out_dtype, accumulate, M, N, K);
  }
}

}  // namespace

// A: [M, K] with row stride lda; W: [N, K] with row stride ldw; out: [M, N]
// with row stride ldo (strides in elements).  accumulate != 0 adds into a
// 32-bit output.
GB_API int gb_linear_simt(const void* A, int a_dtype, long long lda, const void* W, int w_dtype, long long ldw,
                          const float* bias, void* out, int out_dtype, long long ldo, int accumulate, int M, int N,
                          int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return GB_OK;
  if (K <= 0) GB_FAIL(GB_ERR_ARG, "gb_linear_simt: K = %d", K);
  if (accumulate && out_dtype != GB_F32)
    GB_FAIL(GB_ERR_ARG, "gb_linear_simt: accumulation needs a 32-bit output");
  if (out_dtype != GB_F32 && out_dtype != GB_BF16) GB_FAIL(GB_ERR_ARG, "gb_linear_simt: output dtype %d", out_dtype);
  if (gb_div_up(M, 16) > 65535 || gb_div_up(N, 16) > 2147483647LL)
    GB_FAIL(GB_ERR_ARG, "gb_linear_simt: M = %d or N = %d is too large", M, N);
  if (a_dtype == GB_F32 && w_dtype == GB_F32)
    launch<float, float>(A, lda, W, ldw, bias, out, ldo, out_dtype, accumulate, M, N, K, stream);
  else if (a_dtype == GB_BF16 && w_dtype == GB_BF16)
    launch<bf16, bf16>(A, lda, W, ldw, bias, out, ldo, out_dtype, accumulate, M, N, K, stream);
  else if (a_dtype == GB_BF16 && w_dtype == GB_F32)
    launch<bf16, float>(A, lda, W, ldw, bias, out, ldo, out_dtype, accumulate, M, N, K, stream);
  else if (a_dtype == GB_F32 && w_dtype == GB_BF16)
    launch<float, bf16>(A, lda, W, ldw, bias, out, ldo, out_dtype, accumulate, M, N, K, stream);
  else
    GB_FAIL(GB_ERR_ARG, "gb_linear_simt: operand dtypes %d, %d", a_dtype, w_dtype);
  GB_CHECK_LAUNCH("gb_linear_simt");
  return GB_OK;
}
