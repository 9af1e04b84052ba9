// out[m, n] (+)= sum_k X[m, k] * W[n, k] (+ bias[n]) in bfloat16 on the 5th
// generation tensor cores: tcgen05.mma with both operands staged in shared
// memory by TMA (128-byte swizzle) and the 32-bit accumulator in tensor memory.
//
// The weight matrix is always the 128-row side of the instruction and the
// tokens are its N side (16 to 256 columns), so the same kernel serves a
// single decoded token and a 2,048-token prompt: D[n, m] = W[n, :] . X[m, :],
// stored transposed.  One CTA computes one 128 x BN tile over a range of K:
//   warp 0   one elected thread issues the TMA loads (producer),
//   warp 1   allocates tensor memory; one elected thread issues the MMAs,
//   warps 2-5 read the accumulator back (tcgen05.ld) and store the tile.
// When there are too few tiles to fill the GPU (decode), K is split across
// CTAs; the partial tiles go to a 32-bit workspace and a second kernel adds
// them in a fixed order, so results do not depend on timing.
//
// Sizes: any M, N; K a multiple of 8 (16-byte rows for TMA), all row strides
// multiples of 8 elements, 16-byte aligned bases.  Ragged edges are zero-filled
// by TMA on load and masked on store.  Every mbarrier wait is bounded; a wait
// that runs out sets *status and the CTA drains and returns.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;        // weight rows per tile (the M of tcgen05.mma)
constexpr int BK = 64;         // 64 bf16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int W_TILE_BYTES = BM * BK * 2;
constexpr int STATUS_TIMEOUT = 16;

enum OutMode : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2, OUT_PARTIAL = 3 };

template <int BN> struct Cfg {
  static constexpr int X_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
  static constexpr int STAGES = BN >= 256 ? 4 : (BN >= 128 ? 3 : (BN >= 64 ? 4 : 5));
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + room to align to 1024
};

template <int BN>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const float* __restrict__ bias, void* __restrict__ out, long long ldo, int mode, int M, int N,
               int total_kb, int kb_per_split, int* __restrict__ status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[C::STAGES], empty_bar[C::STAGES], tmem_full_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN;
  const int kb_begin = blockIdx.z * kb_per_split;
  const int kb_end = min(kb_begin + kb_per_split, total_kb);
  const int nkb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % C::STAGES;
        const uint32_t ph = (i / C::STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
          abort_flag = 1;
          atomicExch(status, STATUS_TIMEOUT);
          break;
        }
        if (abort_flag) break;
        uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], C::STAGE_BYTES);
        tma_load_2d(st, &tmap_w, (kb_begin + i) * BK, n0, &full_bar[s]);
        tma_load_2d(st + W_TILE_BYTES, &tmap_x, (kb_begin + i) * BK, m0, &full_bar[s]);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % C::STAGES;
        const uint32_t ph = (i / C::STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph)) {
          abort_flag = 1;
          atomicExch(status, STATUS_TIMEOUT + 1);
          break;
        }
        if (abort_flag) break;
        tc_fence_after();
        uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
        const uint64_t da = smem_desc_sw128(st);
        const uint64_t db = smem_desc_sw128(st + W_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // advancing 16 bf16 = 32 bytes inside the swizzled row: +2 in the (address >> 4) field
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (uint32_t)((i | k) != 0));
        }
        umma_commit(&empty_bar[s]);   // frees this stage once the MMAs that read it are done
      }
      umma_commit(&tmem_full_bar);    // the accumulator is complete
    }
    __syncwarp();
  } else {
    const bool ok = mbar_wait(&tmem_full_bar, 0);
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(status, STATUS_TIMEOUT + 2);
    }
    tc_fence_after();
    if (ok && !abort_flag) {
      const int q = warp & 3;                 // this warp may read tensor-memory lanes 32q .. 32q+31
      const int n = n0 + 32 * q + lane;       // the weight row this thread holds
      const float b = (bias != nullptr && mode != OUT_PARTIAL && n < N) ? bias[n] : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (m0 + c0 >= M) break;              // uniform over the warp
        float v[16];
        tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m < M) {
              const float val = v[j] + b;
              if (mode == OUT_BF16) {
                ((bf16*)out)[(size_t)m * ldo + n] = __float2bfloat16_rn(val);
              } else if (mode == OUT_F32) {
                ((float*)out)[(size_t)m * ldo + n] = val;
              } else if (mode == OUT_F32_ACC) {
                float* o = (float*)out + (size_t)m * ldo + n;
                *o = *o + val;
              } else {
                ((float*)out)[((size_t)blockIdx.z * M + m) * (size_t)N + n] = v[j];
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // give copies that are still in flight time to land before the shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// out = sum over splits of the partial tiles (+ bias), in split order.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, const float* __restrict__ bias,
                                     void* __restrict__ out, long long ldo, int mode, int M, int N) {
  const long long total = (long long)M * N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / N), n = (int)(i - (long long)m * N);
    float acc = ws[i];
    for (int s = 1; s < splits; ++s) acc += ws[(size_t)s * total + i];
    if (bias) acc += bias[n];
    const size_t o = (size_t)m * ldo + n;
    if (mode == OUT_BF16) ((bf16*)out)[o] = __float2bfloat16_rn(acc);
    else if (mode == OUT_F32) ((float*)out)[o] = acc;
    else ((float*)out)[o] += acc;
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// A [rows, K] bf16 matrix with row stride ld (elements), read in boxes of box_rows x 64.
bool make_tmap(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct WKey {
  const void* p; long long n, k, ld;
  bool operator==(const WKey& o) const { return p == o.p && n == o.n && k == o.k && ld == o.ld; }
};
struct WKeyHash {
  size_t operator()(const WKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.n) * 31) ^ (std::hash<long long>()(k.k) * 131) ^
           (std::hash<long long>()(k.ld) * 521);
  }
};
std::mutex g_wmap_mutex;
std::unordered_map<WKey, CUtensorMap, WKeyHash> g_wmaps;   // weights do not move: their maps are made once

int pick_bn(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  return 128;
}

void plan(int M, int N, int K, int* bn, int* splits, int* kb_per_split) {
  *bn = pick_bn(M);
  const int total_kb = gb_div_up(K, BK);
  const long long tiles = (long long)gb_div_up(N, BM) * gb_div_up(M, *bn);
  int s = 1;
  if (tiles < 96 && M <= 128) {                  // too few CTAs to pull the weights at full bandwidth
    s = (int)(148 / tiles);
    const int max_by_k = total_kb / 4;           // at least 4 k-blocks (256 columns of K) per split
    if (s > max_by_k) s = max_by_k;
    if (s > 16) s = 16;
    if (s < 1) s = 1;
  }
  *kb_per_split = gb_div_up(total_kb, s);
  *splits = gb_div_up(total_kb, *kb_per_split);
}

template <int BN>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const float* bias, void* out, long long ldo, int mode,
           int M, int N, int total_kb, int kb_per_split, int splits, int* status, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<BN>::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid(gb_div_up(N, BM), gb_div_up(M, BN), splits);
  gemm_tc_kernel<BN><<<grid, 192, Cfg<BN>::SMEM_BYTES, stream>>>(tw, tx, bias, out, ldo, mode, M, N, total_kb,
                                                               kb_per_split, status);
  return GB_OK;
}

}  // namespace

// 32-bit words of workspace gb_linear_tc needs for these sizes (0: none).
GB_API long long gb_linear_tc_workspace(int M, int N, int K) {
  int bn, splits, kbs;
  plan(M, N, K, &bn, &splits, &kbs);
  return splits > 1 ? (long long)splits * M * N : 0;
}

// 1 if gb_linear_tc takes these operands, else 0 (the caller then uses the CUDA-core kernel).
GB_API int gb_linear_tc_supported(const void* X, long long ldx, const void* W, long long ldw, int K) {
  return (K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0)
             ? 1 : 0;
}

// X: [M, K] bf16 (row stride ldx), W: [N, K] bf16 (row stride ldw), bias: f32 [N] or null,
// out: [M, N] bf16 or f32 (row stride ldo); accumulate adds into an f32 out.
// workspace: gb_linear_tc_workspace(M, N, K) floats (may be null when that is 0).
// Returns the number of kernels launched (1 or 2), or a negative error code.
GB_API int gb_linear_tc(const void* X, long long ldx, const void* W, long long ldw, const float* bias, void* out,
                        int out_dtype, long long ldo, int accumulate, int M, int N, int K, float* workspace,
                        int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!gb_linear_tc_supported(X, ldx, W, ldw, K))
    GB_FAIL(GB_ERR_ARG, "gb_linear_tc: K = %d and the row strides (%lld, %lld) must be multiples of 8 and the bases "
            "16-byte aligned", K, ldx, ldw);
  if (accumulate && out_dtype != GB_F32) GB_FAIL(GB_ERR_ARG, "gb_linear_tc: accumulation needs a 32-bit output");
  if (out_dtype != GB_F32 && out_dtype != GB_BF16) GB_FAIL(GB_ERR_ARG, "gb_linear_tc: output dtype %d", out_dtype);
  if (gb_div_up(M, 16) > 65535) GB_FAIL(GB_ERR_ARG, "gb_linear_tc: M = %d is too large", M);
  int bn, splits, kb_per_split;
  plan(M, N, K, &bn, &splits, &kb_per_split);
  if (splits > 1 && workspace == nullptr) GB_FAIL(GB_ERR_ARG, "gb_linear_tc: these sizes need a workspace");

  CUtensorMap tw, tx;
  {
    std::lock_guard<std::mutex> lock(g_wmap_mutex);
    WKey key{W, N, K, ldw};
    auto it = g_wmaps.find(key);
    if (it == g_wmaps.end()) {
      if (!make_tmap(&tw, W, N, K, ldw, BM)) GB_FAIL(GB_ERR_CUDA, "gb_linear_tc: cuTensorMapEncodeTiled failed (W)");
      g_wmaps.emplace(key, tw);
    } else {
      tw = it->second;
    }
  }
  if (!make_tmap(&tx, X, M, K, ldx, bn)) GB_FAIL(GB_ERR_CUDA, "gb_linear_tc: cuTensorMapEncodeTiled failed (X)");

  const int final_mode = out_dtype == GB_BF16 ? OUT_BF16 : (accumulate ? OUT_F32_ACC : OUT_F32);
  const int mode = splits > 1 ? OUT_PARTIAL : final_mode;
  void* dst = splits > 1 ? (void*)workspace : out;
  const int total_kb = gb_div_up(K, BK);
  int rc;
  switch (bn) {
    case 16: rc = launch<16>(tw, tx, bias, dst, ldo, mode, M, N, total_kb, kb_per_split, splits, status, stream); break;
    case 32: rc = launch<32>(tw, tx, bias, dst, ldo, mode, M, N, total_kb, kb_per_split, splits, status, stream); break;
    case 64: rc = launch<64>(tw, tx, bias, dst, ldo, mode, M, N, total_kb, kb_per_split, splits, status, stream); break;
    default: rc = launch<128>(tw, tx, bias, dst, ldo, mode, M, N, total_kb, kb_per_split, splits, status, stream); break;
  }
  if (rc != GB_OK) return rc;
  GB_CHECK_LAUNCH("gb_linear_tc");
  if (splits > 1) {
    const long long total = (long long)M * N;
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(workspace, splits, bias, out, ldo, final_mode, M, N);
    GB_CHECK_LAUNCH("gb_linear_tc (split-K reduce)");
    return 2;
  }
  return 1;
}

// Forget the tensor maps of weights (call when weights are freed, so that a
// later allocation at the same address with another shape gets a new map).
GB_API void gb_linear_tc_forget() {
  std::lock_guard<std::mutex> lock(g_wmap_mutex);
  g_wmaps.clear();
}
