// out[m, n] (+)= sum_k X[m, k] * W[n, k] (+ bias[n]) in bfloat16 on the 5th
// generation tensor cores: tcgen05.mma with both operands staged in shared
// memory by TMA (128-byte swizzle) and the 32-bit accumulator in tensor memory.
//
// The weight matrix is always the 128-row side of the instruction and the
// tokens are its N side (16 to 128 columns), so the same kernel serves a
// single decoded token and a 2,048-token prompt: D[n, m] = W[n, :] . X[m, :],
// stored transposed.  One CTA computes one 128 x BN tile over a range of K:
//   warp 0   one elected thread issues the TMA loads (producer),
//   warp 1   allocates tensor memory; one elected thread issues the MMAs,
//   warps 2-5 read the accumulator back (tcgen05.ld) and store the tile.
//
// Epilogues: store bf16 / store f32 / add into an f32 output (the residual
// stream) / SwiGLU, for a weight whose rows alternate in blocks of 64 between
// gate and up: lanes 0-63 of a tile then hold g, lanes 64-127 hold u of the
// same 64 features, and the tile stores (g * sigmoid(g)) * u.
//
// When there are too few tiles to fill the GPU (decoding), K is split across
// CTAs: every CTA writes its partial tile to a 32-bit workspace, and the
// partial tiles are added in split order (so the result does not depend on
// timing) either by a small second kernel here, or, for a product that adds
// into the residual stream, by the normalisation kernel that reads the stream
// next (the caller asks for that with `defer`).
//
// A decode step is bound by streaming the weights once: the weights are read
// with an evict-first L2 hint.  (Asking L2 ahead of time for the next product's weights, or for
// a product's own tiles behind its ring before its dependency is met, was measured in several
// forms: the product that asks gains up to 1.5 us, the small kernels around it lose more to the
// busier memory system; it is not done.)
//
// Sizes: any M, N; K a multiple of 8 (16-byte rows for TMA), all row strides
// multiples of 8 elements, 16-byte aligned bases.  Ragged edges are zero-filled
// by TMA on load and masked on store.  Every mbarrier wait is bounded; a wait
// that runs out sets *status and the CTA drains and returns.
#include <stdlib.h>

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

enum OutMode : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2, OUT_SWIGLU = 3 };

// DEEP (64-token tiles): a launch with no more CTAs than SMs (every decode product but the head)
// has one CTA per SM anyway; it then takes most of the SM's shared memory for its pipeline, so
// that as many weight bytes are on their way as with the narrower tiles.
// Stages of the 16-token tiles (decode batches up to 16): six of 18 KB are the most that leave room
// for two CTAs per SM (the product after this one then fills its ring while this one streams);
// five measured 2.5 % slower a step; more would leave room for one CTA per SM only (ten stages
// that way were measured slower).
#ifndef GB_NARROW_STAGES
#define GB_NARROW_STAGES 6
#endif
template <int BN, bool DEEP = false> struct Cfg {
  static constexpr int X_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
  static constexpr int STAGES = DEEP ? (BN >= 128 ? 6 : (BN >= 64 ? 8 : (BN >= 32 ? 9 : 10)))
                                     : (BN >= 128 ? 3 : (BN >= 64 ? 4 : (BN >= 32 ? 5 : GB_NARROW_STAGES)));
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + room to align to 1024
};

struct GemmParams {
  const float* bias;
  void* out; long long ldo;
  int mode;                     // OutMode
  int M, N;                     // tokens, weight rows (for SwiGLU: 2 * features)
  int total_kb, kb_per_split, splits;
  float* ws;                    // [splits][M][N] partial tiles (splits > 1)
  int bnp;                      // CTA-pair kernel: tokens per tile
  int stream_weights;           // 1: read W with an evict-first L2 hint
  int vec_store;                // 1: out rows are 16-byte aligned (base and row stride)
  int* status;
};

__device__ __forceinline__ float silu_mul(float g, float u) {
  const float sig = 1.0f / (1.0f + expf(-g));
  return (g * sig) * u;
}

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Applies the epilogue to one finished value D[n][m] (n: weight row) and stores it.
__device__ __forceinline__ void store_value(const GemmParams& p, int m, int n, float val) {
  if (p.mode == OUT_BF16) {
    ((bf16*)p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(val);
  } else if (p.mode == OUT_F32) {
    ((float*)p.out)[(size_t)m * p.ldo + n] = val;
  } else {
    float* o = (float*)p.out + (size_t)m * p.ldo + n;
    *o = *o + val;
  }
}

#ifdef GB_GEMM_TRACE
// Debug builds: %globaltimer stamps of the first CTA of every launch of gemm_tc_kernel.
__device__ unsigned long long* g_gemm_trace = nullptr;   // [launch][3 threads][16]
__device__ unsigned int g_gemm_trace_launch = 0;
__device__ __forceinline__ unsigned long long gtimer_g() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define GSTAMP(row, i) do { if (gtrace) gtrace[(row) * 16 + (i)] = gtimer_g(); } while (0)
#else
#define GSTAMP(row, i) do {} while (0)
#endif

template <int BN, bool DEEP>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const GemmParams p) {
  pdl_trigger();   // the kernel after this one may start its prologue now
  using C = Cfg<BN, DEEP>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[C::STAGES], empty_bar[C::STAGES], tmem_full_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(kb_begin + p.kb_per_split, p.total_kb);
  const int nkb = kb_end - kb_begin;
  const int M = p.M, N = p.N;
#ifdef GB_GEMM_TRACE
  __shared__ unsigned int gtrace_slot;
  if (threadIdx.x == 0) gtrace_slot = (blockIdx.x | blockIdx.y | blockIdx.z) == 0 ? atomicAdd(&g_gemm_trace_launch, 1u) : 0xffffffffu;
  __syncthreads();
  unsigned long long* gtrace = (g_gemm_trace && gtrace_slot < 4096u) ? g_gemm_trace + (size_t)gtrace_slot * 48 : nullptr;
  if (threadIdx.x == 0 && gtrace) {
    for (int i = 0; i < 48; ++i) gtrace[i] = 0;
    gtrace[0] = gtimer_g();
    gtrace[14] = gridDim.x * 1000 + gridDim.z;
    gtrace[15] = p.mode;
  }
  __syncthreads();
#endif

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
      uint64_t policy = 0;
      if (p.stream_weights) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
      auto load_w = [&](int i, int s) {
        uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], C::STAGE_BYTES);
        if (p.stream_weights)
          tma_load_2d_hint(st, &tmap_w, (kb_begin + i) * BK, n0, &full_bar[s], policy);
        else
          tma_load_2d(st, &tmap_w, (kb_begin + i) * BK, n0, &full_bar[s]);
      };
      auto load_x = [&](int i, int s) {
        uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
        tma_load_2d(st + W_TILE_BYTES, &tmap_x, (kb_begin + i) * BK, m0, &full_bar[s]);
      };
      // The weights do not depend on the kernels before this one: their first tiles are
      // requested at once.  The activations are read only after those kernels have finished.
      const int head = nkb < C::STAGES ? nkb : C::STAGES;
      for (int i = 0; i < head; ++i) load_w(i, i);
      GSTAMP(0, 1);
      pdl_wait();
      GSTAMP(0, 2);
      for (int i = 0; i < head; ++i) load_x(i, i);
      GSTAMP(0, 3);
      for (int i = head; i < nkb; ++i) {
        const int s = i % C::STAGES;
        const uint32_t ph = (i / C::STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
          abort_flag = 1;
          atomicExch(p.status, STATUS_TIMEOUT);
          break;
        }
        if (abort_flag) break;
        load_w(i, s);
        load_x(i, s);
      }
      GSTAMP(0, 4);
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
          atomicExch(p.status, STATUS_TIMEOUT + 1);
          break;
        }
        if (abort_flag) break;
        if (i == 0) GSTAMP(1, 1);
        if (i == C::STAGES) GSTAMP(1, 2);
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
      GSTAMP(1, 3);
    }
    __syncwarp();
  } else {
    // ---- epilogue warps (threads 64..191) ----
    const int et = threadIdx.x - 64;            // 0..127
    pdl_wait();    // outputs (and the workspace) may still be read by the kernels before this one
    if (et == 0) GSTAMP(2, 1);
    const bool ok = mbar_wait(&tmem_full_bar, 0);
    if (et == 0) GSTAMP(2, 2);
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT + 2);
    }
    tc_fence_after();
    epilogue_barrier();                          // abort_flag is seen by all epilogue threads
    const bool good = !abort_flag;
    const int q = warp & 3;                      // this warp may read tensor-memory lanes 32q .. 32q+31
    const int row = 32 * q + lane;               // lane of the accumulator = weight row within the tile
    const int n = n0 + row;
    const bool split = p.splits > 1;
    if (good && split && BN >= 32 && n0 + BM <= N && (N & 3) == 0 && (((uintptr_t)p.ws) & 15) == 0) {
      // partial tile -> workspace, 64 token rows at a time through shared memory (the pipeline's
      // stages are free once the accumulator is complete): a warp then stores 512 contiguous bytes
      // of one token's row per instruction.  (Stores of 128 bytes each, 8 KB apart, as the lanes
      // hold them, took 2.7 us for a 64-token tile.)
      float* fb = reinterpret_cast<float*>(tiles);                                     // [64][128]
      const int cols = min(BN, M - m0);
#pragma unroll 1
      for (int h0 = 0; h0 < cols; h0 += 64) {
        const int hc = min(64, cols - h0);
#pragma unroll 1
        for (int c0 = 0; c0 < hc; c0 += 32) {
          float v[32];
          tmem_ld_32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(h0 + c0), v);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < hc) fb[(c0 + j) * BM + row] = v[j];
        }
        epilogue_barrier();
        float* dst = p.ws + ((size_t)blockIdx.z * M + m0 + h0) * (size_t)N + n0;
        for (int idx = et; idx < hc * 32; idx += 128) {         // 32 pieces of 4 floats per row
          const int mm = idx >> 5, piece = idx & 31;
          *reinterpret_cast<float4*>(dst + (size_t)mm * N + piece * 4) =
              *reinterpret_cast<const float4*>(fb + mm * BM + piece * 4);
        }
        if (h0 + 64 < cols) epilogue_barrier();
      }
    } else if (good && split) {
      // partial tile -> workspace (a lane is a weight row: a warp's store is 128 contiguous bytes
      // of one token's row).  32 columns per tensor-memory load where the tile has them: the wait
      // for a load is paid once per 32 stores, not once per 16.
      float* wsp = p.ws + ((size_t)blockIdx.z * M + m0) * (size_t)N + n;
      constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CH) {
        if (m0 + c0 >= M) break;
        float v[CH];
        if (CH == 32) tmem_ld_32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        else tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        if (n < N) {
          const int jmax = min(CH, M - m0 - c0);
#pragma unroll
          for (int j = 0; j < CH; ++j)
            if (j < jmax) wsp[(size_t)(c0 + j) * N] = v[j];
        }
      }
    } else if (good && BN >= 32 && p.vec_store && n0 + BM <= N) {
      // Large tiles: the accumulator is transposed through shared memory (the pipeline's
      // stages are free once the accumulator is complete) and leaves in 16-byte pieces,
      // whole rows of the output at a time, instead of one element per thread and column.
      const float b = p.bias ? p.bias[n] : 0.f;
      const int cols = min(BN, M - m0);                      // token rows of this tile
      if (p.mode == OUT_SWIGLU) {
        // g (accumulator rows 0-63) and u (rows 64-127) go to shared memory in 32-bit; then all
        // 128 threads share the activations, four features of one token at a time, with the fast
        // exponential and division (the result is rounded to bfloat16, which hides both) and
        // store 8 bytes each: sixteen threads write the 128 bytes of a token's 64 features.
        float* gs = reinterpret_cast<float*>(tiles);                                   // [BN][64] g + bias
        float* us = gs + BN * 64;                                                      // [BN][64] u + bias
        float* mine = row < 64 ? gs + row : us + (row - 64);
        constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
        for (int c0 = 0; c0 < cols; c0 += CH) {
          float v[CH];
          if (CH == 32) tmem_ld_32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
          else tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
#pragma unroll
          for (int j = 0; j < CH; ++j)
            if (c0 + j < cols) mine[(c0 + j) * 64] = v[j] + b;
        }
        epilogue_barrier();
        bf16* dst = (bf16*)p.out + (size_t)m0 * p.ldo + (n0 >> 1);
        for (int idx = et; idx < cols * 16; idx += 128) {
          const int mm = idx >> 4, f = (idx & 15) * 4;
          const float4 g4 = *reinterpret_cast<const float4*>(gs + mm * 64 + f);
          const float4 u4 = *reinterpret_cast<const float4*>(us + mm * 64 + f);
          const float r0 = __fdividef(g4.x, 1.0f + __expf(-g4.x)) * u4.x;
          const float r1 = __fdividef(g4.y, 1.0f + __expf(-g4.y)) * u4.y;
          const float r2 = __fdividef(g4.z, 1.0f + __expf(-g4.z)) * u4.z;
          const float r3 = __fdividef(g4.w, 1.0f + __expf(-g4.w)) * u4.w;
          __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
          uint2 packed;
          packed.x = *reinterpret_cast<uint32_t*>(&lo);
          packed.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(dst + (size_t)mm * p.ldo + f) = packed;
        }
      } else if (p.mode == OUT_BF16) {
        bf16* ob = reinterpret_cast<bf16*>(tiles);                                     // [BN][128]
#pragma unroll 1
        for (int c0 = 0; c0 < cols; c0 += 16) {
          float v[16];
          tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) ob[(c0 + j) * BM + row] = __float2bfloat16_rn(v[j] + b);
        }
        epilogue_barrier();
        bf16* dst = (bf16*)p.out + (size_t)m0 * p.ldo + n0;
        for (int idx = et; idx < cols * 16; idx += 128) {       // 16 pieces of 8 bf16 per row
          const int mm = idx >> 4, piece = idx & 15;
          *reinterpret_cast<uint4*>(dst + (size_t)mm * p.ldo + piece * 8) =
              *reinterpret_cast<const uint4*>(ob + mm * BM + piece * 8);
        }
      } else {                                                // OUT_F32 / OUT_F32_ACC, 64 token rows at a time
        float* fb = reinterpret_cast<float*>(tiles);                                   // [64][128]
#pragma unroll 1
        for (int h0 = 0; h0 < cols; h0 += 64) {
          const int hc = min(64, cols - h0);
#pragma unroll 1
          for (int c0 = 0; c0 < hc; c0 += 16) {
            float v[16];
            tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(h0 + c0), v);
#pragma unroll
            for (int j = 0; j < 16; ++j) fb[(c0 + j) * BM + row] = v[j] + b;
          }
          epilogue_barrier();
          float* dst = (float*)p.out + (size_t)(m0 + h0) * p.ldo + n0;
          for (int idx = et; idx < hc * 32; idx += 128 * 4) {   // 32 pieces of 4 floats per row, 4 in flight
            float4 nv[4], ov[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int id = idx + u * 128;
              if (id < hc * 32) {
                const int mm = id >> 5, piece = id & 31;
                nv[u] = *reinterpret_cast<const float4*>(fb + mm * BM + piece * 4);
                if (p.mode == OUT_F32_ACC)
                  ov[u] = __ldcg(reinterpret_cast<const float4*>(dst + (size_t)mm * p.ldo + piece * 4));
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int id = idx + u * 128;
              if (id < hc * 32) {
                const int mm = id >> 5, piece = id & 31;
                float4 r = nv[u];
                if (p.mode == OUT_F32_ACC) { r.x += ov[u].x; r.y += ov[u].y; r.z += ov[u].z; r.w += ov[u].w; }
                *reinterpret_cast<float4*>(dst + (size_t)mm * p.ldo + piece * 4) = r;
              }
            }
          }
          epilogue_barrier();
        }
      }
    } else if (good && p.mode == OUT_SWIGLU) {
      // u of one 16-column chunk, padded against bank conflicts, in the pipeline's first stage
      // (free once the accumulator is complete; static shared memory would cost the second CTA
      // of an SM its place)
      float (*ubuf)[17] = reinterpret_cast<float (*)[17]>(tiles);
      const float b = (p.bias && n < N) ? p.bias[n] : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (m0 + c0 >= M) break;
        float v[16];
        tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        const int jmax = min(16, M - m0 - c0);           // token columns that exist (uniform over the CTA)
        if (row >= 64) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < jmax) ubuf[row - 64][j] = v[j] + b;
        }
        epilogue_barrier();
        if (row < 64) {
          // (the fast exponential and division, as in the CTA-pair kernel's epilogue: the result is
          // rounded to bfloat16, which hides both; a decode step waits for these few instructions)
          bf16* o = (bf16*)p.out + (size_t)(m0 + c0) * p.ldo + (n0 >> 1) + row;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < jmax) {
              const float g = v[j] + b;
              o[(size_t)j * p.ldo] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * ubuf[row][j]);
            }
          }
        }
        if (c0 + 16 < BN && m0 + c0 + 16 < M) epilogue_barrier();   // ubuf is rewritten by the next chunk
      }
    } else if (good) {
      const float b = (p.bias != nullptr && n < N) ? p.bias[n] : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (m0 + c0 >= M) break;                // uniform over the warp
        float v[16];
        tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        if (n < N) {
          if (p.mode == OUT_F32_ACC) {
            // read the 16 old values together (16 loads in flight), then add and store
            float* base = (float*)p.out + (size_t)(m0 + c0) * p.ldo + n;
            float old[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) old[j] = (m0 + c0 + j < M) ? __ldcg(base + (size_t)j * p.ldo) : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (m0 + c0 + j < M) base[(size_t)j * p.ldo] = old[j] + (v[j] + b);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + c0 + j;
              if (m < M) store_value(p, m, n, v[j] + b);
            }
          }
        }
      }
    }
  }
  if (threadIdx.x == 64) GSTAMP(2, 3);
  tc_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // give copies that are still in flight time to land before the shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
  if (threadIdx.x == 64) GSTAMP(2, 8);
}

// ---------------------------------------------------------------- CTA-pair kernel (prompts)
// Two CTAs of a cluster (two SMs) compute one 256 x 256 tile with tcgen05.mma.cta_group::2:
// each CTA stages 128 weight rows (its half of A) and 128 token rows (its half of B) per
// k-block, 32 KB for 128 x 256 x 64 multiply-adds of its own, half the shared-memory traffic
// per flop of a lone CTA, so five stages cover the load latency.  The leader (cluster rank 0)
// issues the MMAs for both; its "full" barriers count the bytes of both CTAs' TMA loads, its
// commits release the stages and publish the accumulator in both CTAs.  Each CTA keeps the
// 128 accumulator rows of its own weight rows in its tensor memory (2 x 256 columns, double
// buffered) and runs its own epilogue.  Persistent: one pair per two SMs walks the tiles.
#ifdef GB_PAIR_TRACE
// Debug builds: %globaltimer stamps and waited cycles of the first and the last pair's leader CTA.
__device__ unsigned long long* g_pair_trace = nullptr;   // [launch][2 CTAs][3 threads][8]
__device__ unsigned int g_pair_trace_launch = 0;
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define PSTAMP(i) do { if (trace) trace[i] = gtimer(); } while (0)
#define PWAIT_BEGIN() const long long w0_ = clock64()
#define PWAIT_END(i) do { if (trace) trace[i] += (unsigned long long)(clock64() - w0_); } while (0)
#define PPHASE_BEGIN() long long ph_ = clock64()
#define PPHASE(i) do { const long long now_ = clock64(); if (trace) trace[i] += (unsigned long long)(now_ - ph_); ph_ = now_; } while (0)
#else
#define PPHASE_BEGIN() do {} while (0)
#define PPHASE(i) do {} while (0)
#define PSTAMP(i) do {} while (0)
#define PWAIT_BEGIN() do {} while (0)
#define PWAIT_END(i) do {} while (0)
#endif

struct PairCfg {
  static constexpr int BNP_MAX = 256;                     // most tokens per tile (GemmParams::bnp: 128..256 in steps of 16)
  static constexpr int X_TILE_BYTES = (BNP_MAX / 2) * BK * 2; // room for this CTA's half of the token rows
  static constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
#ifndef GB_PAIR_STAGES
#define GB_PAIR_STAGES 6
#endif
  static constexpr int STAGES = GB_PAIR_STAGES;
  static constexpr int STAGING_BYTES = 32 * 1024;        // 64 token rows in 32-bit, or 128 in bfloat16
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024;
};

__global__ void __launch_bounds__(192)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const GemmParams p) {
  using C = PairCfg;
  const int BNP = p.bnp;                                  // tokens per tile of this launch
  constexpr int ACC_COLS = C::BNP_MAX;                    // tensor-memory columns per accumulator
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[C::STAGES], empty_bar[C::STAGES], tmem_full_bar[2], tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;
  pdl_trigger();

  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = tiles + (size_t)C::STAGES * C::STAGE_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                // 0: leader
  const int M = p.M, N = p.N, nkb = p.total_kb;
  const int tiles_m = (M + BNP - 1) / BNP, tiles_n = (N + 2 * BM - 1) / (2 * BM);
  const int n_tiles = tiles_m * tiles_n;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
#ifdef GB_PAIR_TRACE
  __shared__ unsigned int trace_slot;
  if (threadIdx.x == 0) trace_slot = blockIdx.x == 0 ? atomicAdd(&g_pair_trace_launch, 1u) : 0u;
  __syncthreads();
  unsigned long long* trace = nullptr;
  if (g_pair_trace && rank == 0 && (pair == 0 || pair == n_pairs - 1) &&
      (threadIdx.x == 0 || threadIdx.x == 32 || threadIdx.x == 64)) {
    // the last pair does not know the slot: it uses the launch counter as it finds it (the first
    // pair of the same launch has already bumped it, or will in a moment; good enough for a probe)
    const unsigned int slot = pair == 0 ? trace_slot : (*(volatile unsigned int*)&g_pair_trace_launch) - 1u;
    if (slot < 1024)
      trace = g_pair_trace + ((size_t)slot * 2 + (pair == 0 ? 0 : 1)) * 24 + (threadIdx.x / 32) * 8;
  }
  if (trace) for (int i = 0; i < 8; ++i) trace[i] = 0;
  PSTAMP(0);
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);       // the leader's producer arrives; both CTAs' loads add bytes
      mbar_init(&empty_bar[s], 1);      // one multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);  // one multicast commit
      mbar_init(&tmem_empty_bar[a], 2); // the epilogues of both CTAs (only the leader's copy is used)
    }
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_slot, C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                   // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      PSTAMP(1);
      // The weights do not depend on the kernels before this one: the weight halves of the first
      // tile's first stages are requested at once, the token halves after the wait.
      int ahead = 0;
      if (pair < n_tiles) {
        ahead = nkb < C::STAGES ? nkb : C::STAGES;
        const int n0 = (pair / tiles_m) * 2 * BM + (int)rank * BM;
        for (int i = 0; i < ahead; ++i) {
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[i], 2 * (W_TILE_BYTES + (BNP / 2) * BK * 2));
          tma_load_2d_pair(tiles + (size_t)i * C::STAGE_BYTES, &tmap_w, i * BK, n0, &full_bar[i]);
        }
      }
      PSTAMP(3);
      pdl_wait();
      PSTAMP(2);
      if (pair < n_tiles) {
        const int m0 = (pair % tiles_m) * BNP + (int)rank * (BNP / 2);
        for (int i = 0; i < ahead; ++i)
          tma_load_2d_pair(tiles + (size_t)i * C::STAGE_BYTES + W_TILE_BYTES, &tmap_x, i * BK, m0, &full_bar[i]);
      }
      int it = 0;
      for (int t = pair; t < n_tiles && !abort_flag; t += n_pairs) {
        const int n0 = (t / tiles_m) * 2 * BM + (int)rank * BM;          // this CTA's weight rows
        const int m0 = (t % tiles_m) * BNP + (int)rank * (BNP / 2);      // this CTA's half of the token rows
        for (int i = 0; i < nkb; ++i, ++it) {
          if (it < ahead) continue;                                      // (requested above)
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            abort_flag = 1;
            atomicExch(p.status, STATUS_TIMEOUT + 8);
            break;
          }
          if (abort_flag) break;
          uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * (W_TILE_BYTES + (BNP / 2) * BK * 2));
          tma_load_2d_pair(st, &tmap_w, i * BK, n0, &full_bar[s]);
          tma_load_2d_pair(st + W_TILE_BYTES, &tmap_x, i * BK, m0, &full_bar[s]);
        }
      }
      PSTAMP(4);
    }
    __syncwarp();
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = idesc_bf16_f32(2 * BM, BNP);
      int it = 0, tile_i = 0;
      for (int t = pair; t < n_tiles && !abort_flag; t += n_pairs, ++tile_i) {
        const int a = tile_i & 1;
        {
          PWAIT_BEGIN();
          if (!mbar_wait(&tmem_empty_bar[a], ((tile_i >> 1) & 1) ^ 1)) {
            abort_flag = 1;
            atomicExch(p.status, STATUS_TIMEOUT + 9);
            break;
          }
          PWAIT_END(5);
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(a * ACC_COLS);
        for (int i = 0; i < nkb; ++i, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          {
            PWAIT_BEGIN();
            if (!mbar_wait(&full_bar[s], ph)) {
              abort_flag = 1;
              atomicExch(p.status, STATUS_TIMEOUT + 10);
              break;
            }
            if (it >= C::STAGES) PWAIT_END(6);
          }
          if (it == 0) PSTAMP(1);
          if (abort_flag) break;
          tc_fence_after();
          uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
          const uint64_t da = smem_desc_sw128(st);
          const uint64_t db = smem_desc_sw128(st + W_TILE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, (uint32_t)((i | k) != 0));
          umma_commit_pair(&empty_bar[s]);
        }
        umma_commit_pair(&tmem_full_bar[a]);
        if (tile_i == 0) PSTAMP(2);
      }
      PSTAMP(3);
#ifdef GB_PAIR_TRACE
      if (trace) trace[4] = (unsigned long long)tile_i;
#endif
    }
    __syncwarp();
  } else {
    const int et = threadIdx.x - 64;
    const int q = warp & 3, row = 32 * q + lane;
    pdl_wait();
    int tile_i = 0;
    for (int t = pair; t < n_tiles; t += n_pairs, ++tile_i) {
      const int a = tile_i & 1;
      const int n0 = (t / tiles_m) * 2 * BM + (int)rank * BM, m0 = (t % tiles_m) * BNP;
      const int n = n0 + row;
      PWAIT_BEGIN();
      const bool ok = mbar_wait(&tmem_full_bar[a], (tile_i >> 1) & 1);
      if (tile_i > 0) PWAIT_END(5);
      if (tile_i == 0) PSTAMP(1);
      PSTAMP(3);
      if (!ok) {
        abort_flag = 1;
        if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT + 11);
      }
      tc_fence_after();
      epilogue_barrier();
      if (abort_flag) break;
      const uint32_t acc = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(a * ACC_COLS);
      const int cols = max(0, min(BNP, M - m0));
      const bool fast = p.vec_store && n0 + BM <= N;
      const float b = (p.bias && n < N) ? p.bias[n] : 0.f;
      const bool f32out = p.mode == OUT_F32 || p.mode == OUT_F32_ACC;
      const int RC = (f32out || p.mode == OUT_SWIGLU) ? 64 : 128;   // token rows staged at a time
      for (int h0 = 0; h0 < BNP; h0 += RC) {
        const int hc = max(0, min(RC, cols - h0));
        const bool last = h0 + RC >= BNP;
        if (hc > 0 && fast && p.mode == OUT_SWIGLU) {
          // g (accumulator rows 0-63) and u (rows 64-127) of 64 token rows go to shared memory
          // in 32-bit; then all 128 threads share the 64 x 64 activations, two features each.
          float* gs = reinterpret_cast<float*>(staging);          // [64][64]
          float* us = gs + 64 * 64;                               // [64][64]
          float* mine = row < 64 ? gs + row : us + (row - 64);
#pragma unroll 1
          for (int c0 = 0; c0 < hc; c0 += 32) {
            float v[32];
            tmem_ld_32(acc + (uint32_t)(h0 + c0), v);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < hc) mine[(c0 + j) * 64] = v[j] + b;
          }
          tc_fence_before();
          epilogue_barrier();
          if (last && et == 0) mbar_arrive_leader(&tmem_empty_bar[a]);
          bf16* dst = (bf16*)p.out + (size_t)(m0 + h0) * p.ldo + (n0 >> 1);
          // The epilogue warps are what this product waits for (they issue several times the
          // instructions of everything else in the kernel), so every instruction counts: four
          // features per thread and step, the fast exponential and the fast division (the result
          // is rounded to bfloat16, which hides both).
          for (int idx = et; idx < hc * 16; idx += 128) {
            const int mm = idx >> 4, f = (idx & 15) * 4;
            const float4 g4 = *reinterpret_cast<const float4*>(gs + mm * 64 + f);
            const float4 u4 = *reinterpret_cast<const float4*>(us + mm * 64 + f);
            const float r0 = __fdividef(g4.x, 1.0f + __expf(-g4.x)) * u4.x;
            const float r1 = __fdividef(g4.y, 1.0f + __expf(-g4.y)) * u4.y;
            const float r2 = __fdividef(g4.z, 1.0f + __expf(-g4.z)) * u4.z;
            const float r3 = __fdividef(g4.w, 1.0f + __expf(-g4.w)) * u4.w;
            __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst + (size_t)mm * p.ldo + f) = packed;
          }
          epilogue_barrier();
        } else if (hc > 0 && fast && p.mode == OUT_BF16) {
          bf16* ob = reinterpret_cast<bf16*>(staging);
#pragma unroll 1
          for (int c0 = 0; c0 < hc; c0 += 32) {
            float v[32];
            tmem_ld_32(acc + (uint32_t)(h0 + c0), v);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < hc) ob[(c0 + j) * BM + row] = __float2bfloat16_rn(v[j] + b);
          }
          tc_fence_before();
          epilogue_barrier();
          if (last && et == 0) mbar_arrive_leader(&tmem_empty_bar[a]);
          bf16* dst = (bf16*)p.out + (size_t)(m0 + h0) * p.ldo + n0;
          for (int idx = et; idx < hc * 16; idx += 128) {
            const int mm = idx >> 4, piece = idx & 15;
            *reinterpret_cast<uint4*>(dst + (size_t)mm * p.ldo + piece * 8) =
                *reinterpret_cast<const uint4*>(ob + mm * BM + piece * 8);
          }
          epilogue_barrier();
        } else if (hc > 0 && fast && p.mode == OUT_F32) {
          // A plain 32-bit store needs no staging: a lane is a weight row, so one store of a warp
          // is 128 contiguous bytes of one token's row, a whole line.
          float* dst = (float*)p.out + (size_t)(m0 + h0) * p.ldo + n;
#pragma unroll 1
          for (int c0 = 0; c0 < hc; c0 += 32) {
            float v[32];
            tmem_ld_32(acc + (uint32_t)(h0 + c0), v);
            if (last && c0 + 32 >= hc) {
              tc_fence_before();
              epilogue_barrier();
              if (et == 0) mbar_arrive_leader(&tmem_empty_bar[a]);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < hc) dst[(size_t)(c0 + j) * p.ldo] = v[j] + b;
          }
        } else if (hc > 0 && fast) {
          float* fb = reinterpret_cast<float*>(staging);
          PPHASE_BEGIN();
#pragma unroll 1
          for (int c0 = 0; c0 < hc; c0 += 32) {
            float v[32];
            tmem_ld_32(acc + (uint32_t)(h0 + c0), v);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < hc) fb[(c0 + j) * BM + row] = v[j] + b;
          }
          PPHASE(6);
          tc_fence_before();
          epilogue_barrier();
          PPHASE(0);
          if (last && et == 0) mbar_arrive_leader(&tmem_empty_bar[a]);
          float* dst = (float*)p.out + (size_t)(m0 + h0) * p.ldo + n0;
          for (int idx = et; idx < hc * 32; idx += 128 * 4) {
            float4 nv[4], ov[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int id = idx + u * 128;
              if (id < hc * 32) {
                const int mm = id >> 5, piece = id & 31;
                nv[u] = *reinterpret_cast<const float4*>(fb + mm * BM + piece * 4);
                if (p.mode == OUT_F32_ACC)
                  ov[u] = __ldcg(reinterpret_cast<const float4*>(dst + (size_t)mm * p.ldo + piece * 4));
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int id = idx + u * 128;
              if (id < hc * 32) {
                const int mm = id >> 5, piece = id & 31;
                float4 r = nv[u];
                if (p.mode == OUT_F32_ACC) { r.x += ov[u].x; r.y += ov[u].y; r.z += ov[u].z; r.w += ov[u].w; }
                *reinterpret_cast<float4*>(dst + (size_t)mm * p.ldo + piece * 4) = r;
              }
            }
          }
          PPHASE(7);
          epilogue_barrier();
          PPHASE(0);
        } else {
          // nothing to store from this chunk, a ragged edge or an unaligned output: element by element
          if (hc > 0 && p.mode == OUT_SWIGLU) {
            float* ub = reinterpret_cast<float*>(staging);
#pragma unroll 1
            for (int c0 = 0; c0 < hc; c0 += 16) {
              float v[16];
              tmem_ld_16(acc + (uint32_t)(h0 + c0), v);
              if (row >= 64) {
#pragma unroll
                for (int j = 0; j < 16; ++j) ub[(c0 + j) * 64 + (row - 64)] = v[j] + b;
              }
            }
            epilogue_barrier();
            if (row < 64 && n + 64 < N) {
#pragma unroll 1
              for (int c0 = 0; c0 < hc; c0 += 16) {
                float v[16];
                tmem_ld_16(acc + (uint32_t)(h0 + c0), v);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (c0 + j < hc)
                    ((bf16*)p.out)[(size_t)(m0 + h0 + c0 + j) * p.ldo + (n0 >> 1) + row] =
                        __float2bfloat16_rn(silu_mul(v[j] + b, ub[(c0 + j) * 64 + row]));
              }
            }
          } else if (hc > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < hc; c0 += 16) {
              float v[16];
              tmem_ld_16(acc + (uint32_t)(h0 + c0), v);
              if (n < N) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (c0 + j < hc) store_value(p, m0 + h0 + c0 + j, n, v[j] + b);
              }
            }
          }
          tc_fence_before();
          epilogue_barrier();
          if (last && et == 0) mbar_arrive_leader(&tmem_empty_bar[a]);
        }
      }
      if (tile_i == 0) PSTAMP(2);
      PSTAMP(4);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  cluster_sync_all();                   // nobody leaves while its partner may still use its memory
  if (warp == 1) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
#ifdef GB_PAIR_TRACE
  if (threadIdx.x == 0 && trace) { trace[5] = gtimer(); trace[6] = ((unsigned long long)gridDim.x << 48) | ((unsigned long long)p.M << 32) | ((unsigned long long)p.N << 8) | (unsigned long long)p.mode; trace[7] = (unsigned long long)p.total_kb; }
#endif
}

// out = epilogue(sum over splits of the partial tiles (+ bias)), in split order.
__global__ void splitk_reduce_kernel(const float* ws, int splits, const float* __restrict__ bias,
                                     void* __restrict__ out, long long ldo, int mode, int M, int N) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)M * N;
  const int n_out = mode == OUT_SWIGLU ? N / 2 : N;
  const long long work = (long long)M * n_out;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < work;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / n_out), c = (int)(i - (long long)m * n_out);
    if (mode == OUT_SWIGLU) {
      const int n = (c / 64) * 128 + (c % 64);          // gate row; its up row is 64 further
      float g = 0.f, u = 0.f;
      for (int s = 0; s < splits; ++s) {
        g += ws[(size_t)s * total + (size_t)m * N + n];
        u += ws[(size_t)s * total + (size_t)m * N + n + 64];
      }
      if (bias) {
        g += bias[n];
        u += bias[n + 64];
      }
      ((bf16*)out)[(size_t)m * ldo + c] = __float2bfloat16_rn(silu_mul(g, u));
    } else {
      float acc = 0.f;
      for (int s = 0; s < splits; ++s) acc += ws[(size_t)s * total + (size_t)m * N + c];
      if (bias) acc += bias[c];
      const size_t o = (size_t)m * ldo + c;
      if (mode == OUT_BF16) ((bf16*)out)[o] = __float2bfloat16_rn(acc);
      else if (mode == OUT_F32) ((float*)out)[o] = acc;
      else ((float*)out)[o] += acc;
    }
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

// (256-token tiles on this kernel, one CTA per SM with four stages, were measured for portions of
// 256 and 512 tokens: 1.71 and 1.99 ms a step against 1.41 and 1.81 ms with two CTAs of 128 per SM.)
int pick_bn(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  return 128;
}

// Below this many 256 x 256 tiles the one-tile CTAs take the product (two per SM; they ask L2 for
// twice the bytes per flop, so they lose as soon as the pairs have enough tiles).
// GIBBS_B200_PAIR_MIN_TILES moves the threshold (for comparison runs).
int gb_pair_min() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("GIBBS_B200_PAIR_MIN_TILES"); v = e ? atoi(e) : 32; }
  return v;
}

int gb_pair();

// Tokens per tile of the CTA-pair kernel: 256 at most; fewer (in steps of 16, the instruction's
// grain) when that saves a round of tiles over the 74 pairs or rows of padding.  The cost of a
// k-block is taken as its shared-memory traffic, which is what the kernel was measured to be
// bound by: 32 KB for the weight rows plus 192 bytes per token.
int pick_bnp(int M, int N) {
  static int forced = -1;
  if (forced < 0) { const char* e = getenv("GIBBS_B200_PAIR_BNP"); forced = e ? atoi(e) : 0; }
  if (forced >= 128 && forced <= 256 && forced % 16 == 0) return forced;
  const long long tiles_n = gb_div_up(N, 2 * BM);
  int best = 256;
  long long best_cost = -1;
  for (int bnp = 256; bnp >= 128; bnp -= 16) {
    const long long tiles = tiles_n * gb_div_up(M, bnp);
    const long long rounds = (tiles + 73) / 74;
    const long long cost = rounds * (32768 + 192 * bnp) + 512 * tiles / 74;   // (a little per tile: its epilogue's tail)
    if (best_cost < 0 || cost < best_cost) { best = bnp; best_cost = cost; }
  }
  return best;
}

// Whether the product runs on CTA pairs (256 x 256 tiles; they never split K: with K split four
// ways a pair per tile and split was measured slower than the one-tile CTAs below, at every size).
bool runs_on_pairs(int M, int N) {
  const long long pair_tiles = (long long)gb_div_up(N, 2 * BM) * gb_div_up(M, 256);
  if (pair_tiles < gb_pair_min() || !gb_pair()) return false;
  // From 96 tokens on a single wave of pairs beats the one-tile CTAs (gate+up at 128 tokens: 19 us
  // against 26 us); with several waves of half-empty token tiles it does not (the head: 65 against 60 us).
  // Below 96 tokens (decode batches) a pair gains 8 % alone but the step loses 3 %: a pair holds its SMs'
  // shared and tensor memory whole, so the products before and after it cannot start under it.
  return M >= 192 || (M >= 96 && pair_tiles <= 74);
}

void plan(int M, int N, int K, int* bn, int* splits, int* kb_per_split) {
  *bn = pick_bn(M);
  const int total_kb = gb_div_up(K, BK);
  const long long tiles = (long long)gb_div_up(N, BM) * gb_div_up(M, *bn);
  int s = 1;
  if (tiles < 96 && M <= 128) {   // too few CTAs to pull the weights at full bandwidth
    s = (int)(148 / tiles);
    const int max_by_k = total_kb / 4;           // at least 4 k-blocks (256 columns of K) per split
    if (s > max_by_k) s = max_by_k;
    if (s > 16) s = 16;
    if (s < 1) s = 1;
  } else if (M > 128 && tiles < 148 && (tiles <= 74 || total_kb >= 64) && !runs_on_pairs(M, N)) {
    // Prompt portions of a few hundred tokens against a narrow weight: a CTA alone walks K at the
    // pace of its own loads (about 75 GB/s), so an under-filled launch takes as long as K is deep,
    // whatever the number of tokens.  Split K until two CTAs per SM are busy.
    s = (int)(296 / tiles);
    const int max_by_k = total_kb / 8;           // at least 8 k-blocks (512 columns of K) per split
    if (s > max_by_k) s = max_by_k;
    if (s > 8) s = 8;
    if (s < 1) s = 1;
  }
  *kb_per_split = gb_div_up(total_kb, s);
  *splits = gb_div_up(total_kb, *kb_per_split);
}

// GIBBS_B200_DEEP_PIPELINE=0 keeps one-wave launches on the short pipeline (for comparison runs).
int gb_deep() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("GIBBS_B200_DEEP_PIPELINE");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v;
}

template <int BN, bool DEEP>
int launch_as(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<BN, DEEP>::SMEM_BYTES));
    attr_set = true;
  }
  gb_launch(gemm_tc_kernel<BN, DEEP>, dim3(grid), dim3(192), Cfg<BN, DEEP>::SMEM_BYTES, stream, tw, tx, p);
  return GB_OK;
}

template <int BN>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t stream) {
  dim3 grid(gb_div_up(p.N, BM), gb_div_up(p.M, BN), p.splits);
  if (BN >= 64) {   // (measured: narrower tiles gain nothing from the deeper pipeline and lose the overlap with the next launch)
    static int n_sm = 0;
    if (n_sm == 0) {
      int dev = 0;
      GB_CUDA(cudaGetDevice(&dev));
      GB_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    }
    if ((long long)grid.x * grid.y * grid.z <= n_sm && gb_deep())
      return launch_as<BN, (BN >= 64)>(tw, tx, p, grid, stream);
  }
  return launch_as<BN, false>(tw, tx, p, grid, stream);
}

int launch_pair(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PairCfg::SMEM_BYTES));
    attr_set = true;
  }
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    GB_CUDA(cudaGetDevice(&dev));
    GB_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  }
  const long long tiles = (long long)gb_div_up(p.N, 2 * BM) * gb_div_up(p.M, p.bnp);
  const int pairs = (int)(tiles < n_sm / 2 ? tiles : n_sm / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = PairCfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gb_pdl_enabled() ? 2 : 1;
  GB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel, tw, tx, p));
  return GB_OK;
}

// GIBBS_B200_PAIR=0 keeps prompts off the CTA-pair kernel (for comparison runs).
int gb_pair() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("GIBBS_B200_PAIR");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v;
}

}  // namespace

// 32-bit words of workspace gb_linear_tc needs for these sizes (0: none).
GB_API long long gb_linear_tc_workspace(int M, int N, int K) {
  int bn, splits, kbs;
  plan(M, N, K, &bn, &splits, &kbs);
  return splits > 1 ? (long long)splits * M * N : 0;
}

// Number of K splits gb_linear_tc uses for these sizes.
GB_API int gb_linear_tc_splits(int M, int N, int K) {
  int bn, splits, kbs;
  plan(M, N, K, &bn, &splits, &kbs);
  return splits;
}

// 1 if gb_linear_tc takes these operands, else 0 (the caller then uses the CUDA-core kernel).
GB_API int gb_linear_tc_supported(const void* X, long long ldx, const void* W, long long ldw, int K) {
  return (K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0)
             ? 1 : 0;
}

// X: [M, K] bf16 (row stride ldx), W: [N, K] bf16 (row stride ldw), bias: f32 [N] or null.
// mode 0: out bf16 [M, N]; 1: out f32; 2: out f32 += ; 3: SwiGLU, W rows alternating in blocks of
// 64 between gate and up (N = 2 * features, a multiple of 128), out bf16 [M, N / 2].
// workspace: gb_linear_tc_workspace(M, N, K) floats (may be null when that is 0).
// defer != 0 (modes 0 and 2): when K is split, leave the partial tiles in the workspace
// ([splits][M][N], without bias) for the caller's next kernel to add (mode 0: and to round to
// bfloat16); nothing is written to out.  defer == 2 (mode 2): the same also when K is not split:
// the whole product goes to the workspace as one "partial" tile set, so that a large product into
// the residual stream only stores (the norm that reads the stream next adds it while it reads)
// instead of reading and rewriting 32-bit rows from its epilogue.
// flags bit 0: read the weights with an evict-first hint.
// Returns the number of kernels launched, or a negative error code.
GB_API int gb_linear_tc(const void* X, long long ldx, const void* W, long long ldw, const float* bias, void* out,
                        int mode, long long ldo, int M, int N, int K, float* workspace, int defer,
                        int flags, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!gb_linear_tc_supported(X, ldx, W, ldw, K))
    GB_FAIL(GB_ERR_ARG, "gb_linear_tc: K = %d and the row strides (%lld, %lld) must be multiples of 8 and the bases "
            "16-byte aligned", K, ldx, ldw);
  if (mode < OUT_BF16 || mode > OUT_SWIGLU) GB_FAIL(GB_ERR_ARG, "gb_linear_tc: output mode %d", mode);
  if (mode == OUT_SWIGLU && N % 128 != 0)
    GB_FAIL(GB_ERR_ARG, "gb_linear_tc: the SwiGLU epilogue needs 2 * features = %d to be a multiple of 128", N);
  if (gb_div_up(M, 16) > 65535) GB_FAIL(GB_ERR_ARG, "gb_linear_tc: M = %d is too large", M);
  int bn, splits, kb_per_split;
  plan(M, N, K, &bn, &splits, &kb_per_split);
  if (splits > 1 && workspace == nullptr) GB_FAIL(GB_ERR_ARG, "gb_linear_tc: these sizes need a workspace");
  if (defer && mode != OUT_F32_ACC && mode != OUT_BF16)
    GB_FAIL(GB_ERR_ARG, "gb_linear_tc: only a plain bfloat16 or an accumulating product can be deferred");

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
  const bool pairs = splits == 1 && runs_on_pairs(M, N);    // each CTA of a pair stages half of a tile's token rows
  const int bnp = pairs ? pick_bnp(M, N) : 256;
  if (!make_tmap(&tx, X, M, K, ldx, pairs ? bnp / 2 : bn)) GB_FAIL(GB_ERR_CUDA, "gb_linear_tc: cuTensorMapEncodeTiled failed (X)");

  if (defer == 2 && splits == 1) {
    if (mode != OUT_F32_ACC || workspace == nullptr)
      GB_FAIL(GB_ERR_ARG, "gb_linear_tc: an unsplit product is deferred only when it adds into a 32-bit output and has "
              "a workspace");
    mode = OUT_F32;            // plain stores of the product, without the bias, into the workspace
    out = workspace;
    ldo = N;
    bias = nullptr;
  }
  GemmParams p;
  p.bias = bias; p.out = out; p.ldo = ldo; p.mode = mode; p.M = M; p.N = N;
  p.total_kb = gb_div_up(K, BK); p.kb_per_split = kb_per_split; p.splits = splits;
  p.ws = workspace;
  p.bnp = bnp;
  const bool decode_like = M <= 64;
  p.stream_weights = (decode_like && (flags & 1)) ? 1 : 0;   // flags bit 0: evict-first hint for the weights
  p.vec_store = (((uintptr_t)out & 15) == 0 && (ldo * (mode == OUT_BF16 || mode == OUT_SWIGLU ? 2 : 4)) % 16 == 0) ? 1 : 0;
  p.status = status;
  int rc;
  const long long n_tiles = (long long)gb_div_up(N, BM) * gb_div_up(M, bn);
  if (pairs) {
    rc = launch_pair(tw, tx, p, stream);
  } else {
    switch (bn) {
      case 16: rc = launch<16>(tw, tx, p, stream); break;
      case 32: rc = launch<32>(tw, tx, p, stream); break;
      case 64: rc = launch<64>(tw, tx, p, stream); break;
      default: rc = launch<128>(tw, tx, p, stream); break;
    }
  }
  if (rc != GB_OK) return rc;
  GB_CHECK_LAUNCH("gb_linear_tc");
  if (splits > 1 && !defer) {
    const long long work = (long long)M * (mode == OUT_SWIGLU ? N / 2 : N);
    const int blocks = (int)((work + 255) / 256 < 148 * 8 ? (work + 255) / 256 : 148 * 8);
    gb_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, workspace, splits, bias, out, ldo, mode, M, N);
    GB_CHECK_LAUNCH("gb_linear_tc (split-K reduce)");
    return 2;
  }
  return 1;
}

// Forget the tensor maps of weights.
GB_API void gb_linear_tc_forget() {
  std::lock_guard<std::mutex> lock(g_wmap_mutex);
  g_wmaps.clear();
}

// ---------------------------------------------------------------- no-allocation entry point
// See gb_no_alloc.h.  The split-K partial tiles live in a fixed array inside this
// library instead of a caller-provided workspace.
#include "gb_no_alloc.h"

namespace {

// Every GPU that loads this library holds these 4 MiB until the process exits.
static __device__ __align__(256) float g_static_workspace[GB_NO_ALLOC_MAX_WORKSPACE_FLOATS];

constexpr int MAX_DEVICES = 64;
std::mutex g_static_mutex;
float* g_static_ptr[MAX_DEVICES] = {nullptr};

// The device address of g_static_workspace on the current device.  In host code the
// array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_workspace(float** out) {
  int dev = -1;
  GB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) GB_FAIL(GB_ERR_ARG, "gb_linear_tc_no_alloc: device index %d", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    GB_CUDA(cudaGetSymbolAddress(&p, g_static_workspace));
    g_static_ptr[dev] = (float*)p;
  }
  *out = g_static_ptr[dev];
  return GB_OK;
}

}  // namespace

// What the product will really use of the built-in scratch: 0 also for a product of more than
// 128 rows whose partial tiles would not fit (it runs with K whole).
GB_API long long gb_linear_tc_no_alloc_needs(int M, int N, int K) {
  const long long need = gb_linear_tc_workspace(M, N, K);
  return (M > 128 && need > GB_NO_ALLOC_MAX_WORKSPACE_FLOATS) ? 0 : need;
}

GB_API int gb_linear_tc_no_alloc(const void* X, long long ldx, const void* W, long long ldw, const float* bias,
                                 void* out, int mode, long long ldo, int M, int N, int K, int* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!gb_linear_tc_supported(X, ldx, W, ldw, K))
    GB_FAIL(GB_ERR_ARG, "gb_linear_tc_no_alloc: K = %d and the row strides (%lld, %lld) must be multiples of 8 and "
            "the bases 16-byte aligned", K, ldx, ldw);
  if (mode < OUT_BF16 || mode > OUT_SWIGLU) GB_FAIL(GB_ERR_ARG, "gb_linear_tc_no_alloc: output mode %d", mode);
  if (mode == OUT_SWIGLU && N % 128 != 0)
    GB_FAIL(GB_ERR_ARG, "gb_linear_tc_no_alloc: the SwiGLU epilogue needs N = %d to be a multiple of 128", N);
  if (status == nullptr) GB_FAIL(GB_ERR_ARG, "gb_linear_tc_no_alloc: a status word on the device is required");
  if (gb_div_up(M, 16) > 65535) GB_FAIL(GB_ERR_ARG, "gb_linear_tc_no_alloc: M = %d is too large", M);
  int bn, splits, kb_per_split;
  plan(M, N, K, &bn, &splits, &kb_per_split);
  long long need = splits > 1 ? (long long)splits * M * N : 0;
  if (M > 128 && need > GB_NO_ALLOC_MAX_WORKSPACE_FLOATS) {
    // above 128 rows the split is for speed only: without the scratch for it, K stays whole
    splits = 1;
    kb_per_split = gb_div_up(K, BK);
    need = 0;
  }
  if (need > GB_NO_ALLOC_MAX_WORKSPACE_FLOATS)
    GB_FAIL(GB_ERR_ARG, "gb_linear_tc_no_alloc: M = %d, N = %d, K = %d split K %d ways and need %lld floats of "
            "scratch; the built-in scratch holds %d (use gb_linear_tc with your own workspace)",
            M, N, K, splits, need, GB_NO_ALLOC_MAX_WORKSPACE_FLOATS);
  float* ws = nullptr;
  if (splits > 1) {
    const int rc = static_workspace(&ws);
    if (rc != GB_OK) return rc;
  }
  CUtensorMap tw, tx;   // on the stack: no cache, nothing is kept between calls
  if (!make_tmap(&tw, W, N, K, ldw, BM)) GB_FAIL(GB_ERR_CUDA, "gb_linear_tc_no_alloc: cuTensorMapEncodeTiled failed (W)");
  if (!make_tmap(&tx, X, M, K, ldx, bn)) GB_FAIL(GB_ERR_CUDA, "gb_linear_tc_no_alloc: cuTensorMapEncodeTiled failed (X)");
  GemmParams p;
  p.bias = bias; p.out = out; p.ldo = ldo; p.mode = mode; p.M = M; p.N = N;
  p.total_kb = gb_div_up(K, BK); p.kb_per_split = kb_per_split; p.splits = splits;
  p.ws = ws;
  p.bnp = 256;                  // (the CTA-pair kernel is not used here)
  p.stream_weights = M <= 64 ? 1 : 0;
  p.vec_store = (((uintptr_t)out & 15) == 0 && (ldo * (mode == OUT_BF16 || mode == OUT_SWIGLU ? 2 : 4)) % 16 == 0) ? 1 : 0;
  p.status = status;
  int rc;
  switch (bn) {
    case 16: rc = launch<16>(tw, tx, p, stream); break;
    case 32: rc = launch<32>(tw, tx, p, stream); break;
    case 64: rc = launch<64>(tw, tx, p, stream); break;
    default: rc = launch<128>(tw, tx, p, stream); break;
  }
  if (rc != GB_OK) return rc;
  GB_CHECK_LAUNCH("gb_linear_tc_no_alloc");
  if (splits > 1) {
    const long long work = (long long)M * (mode == OUT_SWIGLU ? N / 2 : N);
    const int blocks = (int)((work + 255) / 256 < 148 * 8 ? (work + 255) / 256 : 148 * 8);
    gb_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)ws, splits, bias, out, ldo, mode,
              M, N);
    GB_CHECK_LAUNCH("gb_linear_tc_no_alloc (split-K reduce)");
    return 2;
  }
  return 1;
}

#ifdef GB_PAIR_TRACE
// Debug builds: where the pair kernel writes its stamps ([1024][2][3][8] 64-bit words), or null.
GB_API int gb_linear_pair_trace(unsigned long long* buffer) {
  unsigned int zero = 0;
  GB_CUDA(cudaMemcpyToSymbol(g_pair_trace, &buffer, sizeof(buffer)));
  GB_CUDA(cudaMemcpyToSymbol(g_pair_trace_launch, &zero, sizeof(zero)));
  return GB_OK;
}
#endif

#ifdef GB_GEMM_TRACE
// Debug builds: where gemm_tc_kernel writes its stamps ([4096][3][16] 64-bit words), or null.
GB_API int gb_linear_tc_trace(unsigned long long* buffer) {
  unsigned int zero = 0;
  GB_CUDA(cudaMemcpyToSymbol(g_gemm_trace, &buffer, sizeof(buffer)));
  GB_CUDA(cudaMemcpyToSymbol(g_gemm_trace_launch, &zero, sizeof(zero)));
  return GB_OK;
}
#endif
