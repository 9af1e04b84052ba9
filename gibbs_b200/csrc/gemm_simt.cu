// out[m, n] (+)= sum_k A[m, k] * W[n, k] (+ bias[n]) with 32-bit FMA on the CUDA
// cores: the matrix product of the true 32-bit path, and of any operand pair
// the tensor-core kernel does not take (a weight kept in 32-bit beside 16-bit
// activations, sizes it refuses).  No tensor-core mode of any kind is used.
//
// Each output element is one accumulator that walks k in ascending order, so
// its value does not depend on the tile shape or on the rows beside it.
// (MisterTK/gibbs Linear: src/graph/cpu.rs:249-274, 2338-2417.)
#include "common.cuh"

namespace {

constexpr int BN = 64;
constexpr int BK = 16;

template <typename TA, typename TW, int TM>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, long long lda, const TW* __restrict__ W, long long ldw,
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
      const size_t o = (size_t)gm * ldo + gn;
      if (out_dtype == GB_F32) {
        float* of = (float*)out;
        of[o] = accumulate ? of[o] + v : v;
      } else {
        ((bf16*)out)[o] = __float2bfloat16_rn(v);
      }
    }
  }
}

template <typename TA, typename TW>
void launch(const void* A, long long lda, const void* W, long long ldw, const float* bias, void* out, long long ldo,
            int out_dtype, int accumulate, int M, int N, int K, cudaStream_t stream) {
  if (M <= 16) {
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
  if (gb_div_up(M, 16) > 65535) GB_FAIL(GB_ERR_ARG, "gb_linear_simt: M = %d is too large", M);
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
