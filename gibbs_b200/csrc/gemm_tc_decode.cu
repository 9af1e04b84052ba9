// Matrix products of decode steps (up to 64 tokens): out[m, n] (+)= sum_k X[m, k] * W[n, k].
//
// A decode step is a chain of some sixty such products, each of which streams its weight
// once and has almost nothing else to do; what the chain costs beyond the weight stream are
// the kernels between the products.  This kernel takes two of them in:
//
//  * Split K inside a thread-block cluster.  When a weight has too few 128-row tiles to
//    occupy the GPU, the CTAs of one cluster (up to 8, along grid z) each walk a range of K
//    for the same tile.  Afterwards every CTA owns a slice of the tile's rows: each CTA sends
//    the other slices of its partial accumulator into the owners' shared memory (distributed
//    shared memory, plain st.shared::cluster stores), one cluster barrier follows, and each
//    owner adds the partial slices in rank order and runs the epilogue for its rows.  No
//    partial tile goes through global memory and no second kernel adds them; the sum does
//    not depend on timing.
//
//  * RMSNorm in front of the product (up to 16 rows).  With x_mode 1 the token operand is
//    not read by TMA: the four epilogue warps, idle during the main loop, read the 32-bit
//    residual rows, scale them by rsqrt(mean(x^2) + eps) * gain and write the bfloat16
//    operand tiles of the CTA's whole K range into shared memory (in the 128-byte swizzle
//    the MMA expects), eight k-blocks at a time, each group announced on a barrier of its
//    own so that the MMAs start on the first while the later ones are written.  The sum of
//    squares of a row comes as partial sums that the product before left (mode RESIDUAL
//    below), or is taken here when there are none.
//
// Epilogues: bf16 / f32 store, SwiGLU (weight rows alternating in blocks of 64 between gate
// and up), and RESIDUAL: x[m, n] += product (+ bias) on the 32-bit stream, leaving per
// (tile, rank) partial sums of squares of the new rows for the norm of the next product.
//
// Roles in a CTA as in gemm_tc.cu: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 operand
// producers (x_mode 1) and epilogue.  Every mbarrier wait is bounded; a wait that runs out
// sets *status, and the CTA still takes part in the cluster barrier before it returns.
#include <stdlib.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int W_TILE_BYTES = BM * BK * 2;
constexpr int STATUS_TIMEOUT = 32;
constexpr int MAX_CLUSTER = 8;
constexpr int XBUF_ROWS = BM + 2 * (MAX_CLUSTER - 1) + 2;    // slices of ceil(rows / ranks) rows, two halves
constexpr int XN_ROWS = 16;          // x_mode 1 takes up to this many rows
constexpr int XN_GROUP = 8;          // k-blocks per group of operand tiles announced together
constexpr int XN_MAX_KB = 32;        // k-blocks of one CTA whose operand tiles stay in shared memory
constexpr int XN_TILE_BYTES = XN_ROWS * BK * 2;

enum DOut : int { D_BF16 = 0, D_F32 = 1, D_RESIDUAL = 2, D_SWIGLU = 3 };

template <int BN> struct DCfg {
  static constexpr int X_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
  static constexpr int STAGES = BN >= 64 ? 6 : 5;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int XBUF_BYTES = XBUF_ROWS * BN * 4;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + XBUF_BYTES + 1024;
};

struct DecodeParams {
  // token operand
  int x_mode;                    // 0: bf16 rows by TMA; 1: 32-bit rows, normalised here
  const float* xn; long long ldxn;   // x_mode 1: the residual rows
  const float* gain; float eps;
  const int* rows;               // x_mode 1: row m of the product is row rows[m] of xn (null: m)
  const float* ssq_in; int ssq_in_parts; long long ssq_in_ld;   // partial sums of squares [parts][ld], or null
  int K;
  // output
  const float* bias;
  void* out; long long ldo;
  int mode;
  int M, N;
  int total_kb, kb_per_split, splits;
  float* ssq_out; long long ssq_out_ld;
  int stream_weights;
  int* status;
};

__device__ __forceinline__ float silu_mul(float g, float u) {
  const float sig = 1.0f / (1.0f + expf(-g));
  return (g * sig) * u;
}

__device__ __forceinline__ void producer_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

#ifdef GB_DECODE_TRACE
__device__ unsigned long long* g_trace = nullptr;   // [launch][cta 0 / last][16] globaltimer stamps (debug builds)
__device__ unsigned int g_trace_launch = 0;
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define STAMP(i) do { if (trace) trace[i] = gtimer(); } while (0)
#else
#define STAMP(i) do {} while (0)
#endif

template <int BN>
__global__ void __launch_bounds__(192, 2)
gemm_tc_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const DecodeParams p) {
  pdl_trigger();
  using C = DCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[C::STAGES], empty_bar[C::STAGES], tmem_full_bar, x_ready[XN_MAX_KB / XN_GROUP];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;
  __shared__ float xscale[BN];

  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* xbuf = reinterpret_cast<float*>(tiles + (size_t)C::STAGES * C::STAGE_BYTES);
  uint8_t* xres = tiles + (size_t)C::STAGES * C::STAGE_BYTES + C::XBUF_BYTES;   // x_mode 1: [nkb][16 x 64] bf16
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();            // == blockIdx.z: clusters are (1, 1, splits)
  const int S = p.splits;
  const int n0 = blockIdx.x * BM;
  const int kb_begin = rank * p.kb_per_split;
  const int kb_end = min(kb_begin + p.kb_per_split, p.total_kb);
  const int nkb = kb_end - kb_begin;
  const int M = p.M, N = p.N;
  const bool xn_mode = p.x_mode != 0;
  const bool direct = S == 1 && p.mode != D_RESIDUAL;     // every thread stores its own row of the tile itself
#ifdef GB_DECODE_TRACE
  __shared__ unsigned int trace_slot;
  if (threadIdx.x == 0 && blockIdx.x == 0 && rank == 0) trace_slot = atomicAdd(&g_trace_launch, 1u);
  __syncthreads();
  unsigned long long* trace = nullptr;
  if (g_trace && blockIdx.x == 0 && rank == 0 && trace_slot < 4096 && (threadIdx.x == 0 || threadIdx.x == 32 || threadIdx.x == 64))
    trace = g_trace + (size_t)trace_slot * 48 + (threadIdx.x / 32) * 16;
  STAMP(0);
  if (trace && threadIdx.x == 0) { trace[14] = gridDim.x * 1000 + S; trace[15] = xn_mode * 10 + p.mode; }
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int g = 0; g < XN_MAX_KB / XN_GROUP; ++g) mbar_init(&x_ready[g], 128);
    mbar_init(&tmem_full_bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    if (!xn_mode) tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  float old_x[2] = {0.f, 0.f};                   // RESIDUAL: what this thread's outputs are added to

  if (warp == 0) {
    if (elect_one()) {
      uint64_t policy = 0;
      if (p.stream_weights) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
      const uint32_t tx = xn_mode ? W_TILE_BYTES : C::STAGE_BYTES;
      auto load_w = [&](int i, int s) {
        uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], tx);
        if (p.stream_weights)
          tma_load_2d_hint(st, &tmap_w, (kb_begin + i) * BK, n0, &full_bar[s], policy);
        else
          tma_load_2d(st, &tmap_w, (kb_begin + i) * BK, n0, &full_bar[s]);
      };
      auto load_x = [&](int i, int s) {
        uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
        tma_load_2d(st + W_TILE_BYTES, &tmap_x, (kb_begin + i) * BK, 0, &full_bar[s]);
      };
      // the weights do not depend on the kernels before this one
      const int head = nkb < C::STAGES ? nkb : C::STAGES;
      for (int i = 0; i < head; ++i) load_w(i, i);
      STAMP(1);
      if (!xn_mode) {
        pdl_wait();
        STAMP(2);
        for (int i = 0; i < head; ++i) load_x(i, i);
      }
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
        if (!xn_mode) load_x(i, s);
      }
      STAMP(3);
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
        if (xn_mode && i % XN_GROUP == 0 && !mbar_wait(&x_ready[i / XN_GROUP], 0)) {
          abort_flag = 1;
          atomicExch(p.status, STATUS_TIMEOUT + 4);
          break;
        }
        tc_fence_after();
        uint8_t* st = tiles + (size_t)s * C::STAGE_BYTES;
        const uint64_t da = smem_desc_sw128(st);
        const uint64_t db = smem_desc_sw128(xn_mode ? xres + (size_t)i * XN_TILE_BYTES : st + W_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (uint32_t)((i | k) != 0));
        umma_commit(&empty_bar[s]);
      }
      umma_commit(&tmem_full_bar);
      STAMP(2);
    }
    __syncwarp();
  } else {
    const int pw = warp - 2;                     // 0..3
    pdl_wait();                                  // inputs, outputs and the stream may still be in use before this
    STAMP(1);
    // a product into the stream reads what it adds to as early as it can (not after the main loop)
    const int et0 = threadIdx.x - 64;
    if (p.mode == D_RESIDUAL) {
      // (the mapping of the epilogue below: token c = thread mod a power of two, rows thread / that, + k * step)
      const int lg = M <= 1 ? 0 : (M <= 2 ? 1 : (M <= 4 ? 2 : (M <= 8 ? 3 : (M <= 16 ? 4 : (M <= 32 ? 5 : 6)))));
      const int rows_per = (BM + S - 1) / S;
      const int rows_mine = max(0, min(rows_per, BM - rank * rows_per));
      const int c = et0 & ((1 << lg) - 1), r0 = et0 >> lg, rstep = 128 >> lg;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = r0 + u * rstep, n = n0 + rank * rows_per + r;
        if (c < M && r < rows_mine && n < N) old_x[u] = __ldcg((const float*)p.out + (size_t)c * p.ldo + n);
      }
    }
    if (xn_mode) {
      // ---- operand tiles of the CTA's whole K range, eight k-blocks at a time.  The rows' loads of
      // the first group go out before the sums of squares are fetched, so that both travel together.
      constexpr int PER_PASS = 4;                // pieces of 8 columns per thread whose loads are in flight together
      // a piece is 8 columns of one row of one k-block; pieces are numbered (k-block, row, 8 columns)
      // with the rows padded to a power of two, so that no division is needed to find one's piece
      const int lgm = M <= 1 ? 0 : (M <= 2 ? 1 : (M <= 4 ? 2 : (M <= 8 ? 3 : 4)));
      auto piece = [&](int idx, int& m, int& kb, int& c) {
        c = idx & 7;
        m = (idx >> 3) & ((1 << lgm) - 1);
        kb = idx >> (3 + lgm);
      };
      // Registers for two passes: the loads of the next pass are under way while this one is
      // scaled and stored.
      float4 xv[2][PER_PASS][2], gv[2][PER_PASS][2];
      auto load_pass = [&](auto bufc, int g, int idx0) {
        constexpr int buf = decltype(bufc)::value;
        const int kb0 = g * XN_GROUP, kbs = min(XN_GROUP, nkb - kb0);
#pragma unroll
        for (int u = 0; u < PER_PASS; ++u) {
          const int idx = idx0 + u * 128 + et0;
          int m, kb, c;
          piece(idx, m, kb, c);
          const int k = (kb_begin + kb0 + kb) * BK + c * 8;
          if (kb < kbs && m < M && k < p.K) {
            const long long sr = p.rows ? p.rows[m] : m;
            const float4* src = reinterpret_cast<const float4*>(p.xn + (size_t)sr * p.ldxn + k);
            xv[buf][u][0] = __ldcg(src);
            xv[buf][u][1] = __ldcg(src + 1);
            const float4* gs = reinterpret_cast<const float4*>(p.gain + k);
            gv[buf][u][0] = __ldg(gs);
            gv[buf][u][1] = __ldg(gs + 1);
          } else {
            xv[buf][u][0] = xv[buf][u][1] = gv[buf][u][0] = gv[buf][u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      };
      auto store_pass = [&](auto bufc, int g, int idx0) {
        constexpr int buf = decltype(bufc)::value;
        const int kb0 = g * XN_GROUP, kbs = min(XN_GROUP, nkb - kb0);
#pragma unroll
        for (int u = 0; u < PER_PASS; ++u) {
          const int idx = idx0 + u * 128 + et0;
          int m, kb, c;
          piece(idx, m, kb, c);
          if (kb < kbs && m < M) {
            const float sc = xscale[m];
            const float4 x0 = xv[buf][u][0], x1 = xv[buf][u][1], g0 = gv[buf][u][0], g1 = gv[buf][u][1];
            __nv_bfloat162 b0 = __floats2bfloat162_rn(x0.x * sc * g0.x, x0.y * sc * g0.y);
            __nv_bfloat162 b1 = __floats2bfloat162_rn(x0.z * sc * g0.z, x0.w * sc * g0.w);
            __nv_bfloat162 b2 = __floats2bfloat162_rn(x1.x * sc * g1.x, x1.y * sc * g1.y);
            __nv_bfloat162 b3 = __floats2bfloat162_rn(x1.z * sc * g1.z, x1.w * sc * g1.w);
            uint4 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&b0);
            packed.y = *reinterpret_cast<uint32_t*>(&b1);
            packed.z = *reinterpret_cast<uint32_t*>(&b2);
            packed.w = *reinterpret_cast<uint32_t*>(&b3);
            // 128-byte swizzle: the 16-byte piece c of row m lies at piece (c ^ (m & 7))
            *reinterpret_cast<uint4*>(xres + (size_t)(kb0 + kb) * XN_TILE_BYTES + m * 128 + ((c ^ (m & 7)) << 4)) = packed;
          }
        }
      };
      const int n_groups = (nkb + XN_GROUP - 1) / XN_GROUP;
      using B0 = std::integral_constant<int, 0>;
      using B1 = std::integral_constant<int, 1>;
      load_pass(B0{}, 0, 0);
      // ---- the norm's scale per row: from the partial sums the product before left, or from the row
      // itself.  A warp takes rows pw, pw + 4, ...; the loads of all its rows go out together.
      {
        float ss[XN_ROWS / 4];
#pragma unroll
        for (int j = 0; j < XN_ROWS / 4; ++j) {
          const int m = pw + 4 * j;
          ss[j] = 0.f;
          if (m < M) {
            const long long sr = p.rows ? p.rows[m] : m;
            if (p.ssq_in) {
              // eight loads in flight per lane (a loop that adds as it loads would wait for each in turn)
              for (int q0 = 0; q0 < p.ssq_in_parts; q0 += 256) {
                float t[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                  const int q = q0 + u * 32 + lane;
                  t[u] = q < p.ssq_in_parts ? __ldcg(p.ssq_in + (size_t)q * p.ssq_in_ld + sr) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) ss[j] += t[u];
              }
            } else {
              const float4* src = reinterpret_cast<const float4*>(p.xn + (size_t)sr * p.ldxn);
              for (int c0 = 0; c0 < (p.K >> 2); c0 += 256) {
                float4 t[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                  const int c = c0 + u * 32 + lane;
                  t[u] = c < (p.K >> 2) ? __ldcg(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) ss[j] += t[u].x * t[u].x + t[u].y * t[u].y + t[u].z * t[u].z + t[u].w * t[u].w;
              }
            }
          }
        }
#pragma unroll
        for (int j = 0; j < XN_ROWS / 4; ++j) {
          const int m = pw + 4 * j;
          const float t = warp_sum(ss[j]);
          if (lane == 0 && m < M) xscale[m] = 1.0f / sqrtf(t / (float)p.K + p.eps);
        }
      }
      producer_barrier();
      STAMP(2);
      int buf = 0;
      for (int g = 0; g < n_groups; ++g) {
        const int kbs = min(XN_GROUP, nkb - g * XN_GROUP);
        const int total = (kbs * 8) << lgm;
        for (int idx0 = 0; idx0 < total; idx0 += 128 * PER_PASS) {
          // the pass after this one: the rest of this group, or the start of the next
          const bool more = idx0 + 128 * PER_PASS < total;
          const int ng = more ? g : g + 1, nidx = more ? idx0 + 128 * PER_PASS : 0;
          if (buf == 0) {
            if (ng < n_groups) load_pass(B1{}, ng, nidx);
            store_pass(B0{}, g, idx0);
          } else {
            if (ng < n_groups) load_pass(B0{}, ng, nidx);
            store_pass(B1{}, g, idx0);
          }
          buf ^= 1;
        }
        fence_proxy_async();                     // these writes are read by the tensor core (async proxy)
        mbar_arrive(&x_ready[g]);
        if (g == 0) STAMP(3);
      }
      STAMP(4);
    }
    // ---- the accumulator
    const bool ok = mbar_wait(&tmem_full_bar, 0);
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT + 2);
    }
    tc_fence_after();
    STAMP(5);
    producer_barrier();
    const int q = warp & 3;                      // this warp may read tensor-memory lanes 32q .. 32q+31
    const int row = 32 * q + lane;
    if (!abort_flag && direct) {
      // One CTA has the whole K: every thread finishes its own row of the tile (the code on this
      // path is counted in instructions: a single warp runs a dependent chain at a few hundred
      // instructions a microsecond, and the kernel after this one waits for it).
      const int n = n0 + row;
      const float b = (p.bias != nullptr && n < N) ? p.bias[n] : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (c0 >= M) break;
        float v[16];
        tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        if (p.mode == D_SWIGLU) {
          if (row >= 64) {
#pragma unroll
            for (int j = 0; j < 16; ++j) xbuf[(row - 64) * 17 + j] = v[j] + b;
          }
          producer_barrier();
          if (row < 64) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < M)
                ((bf16*)p.out)[(size_t)(c0 + j) * p.ldo + (n0 >> 1) + row] =
                    __float2bfloat16_rn(silu_mul(v[j] + b, xbuf[row * 17 + j]));
          }
          producer_barrier();
        } else if (n < N) {
          if (p.mode == D_BF16) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < M) ((bf16*)p.out)[(size_t)(c0 + j) * p.ldo + n] = __float2bfloat16_rn(v[j] + b);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < M) ((float*)p.out)[(size_t)(c0 + j) * p.ldo + n] = v[j] + b;
          }
        }
      }
    } else if (!abort_flag) {
      // every row's values go to the CTA of the cluster that owns the row
      const int H = p.mode == D_SWIGLU ? 2 : 1;
      const int half_rows = BM / H;
      const int rows_per = (half_rows + S - 1) / S;
      const int hrow = H == 2 ? (row & 63) : row, half = H == 2 ? (row >> 6) : 0;
      const int owner = hrow / rows_per, r = hrow - owner * rows_per;
      const uint32_t offset = (uint32_t)((((rank * H + half) * rows_per + r) * BN) * 4);
      float* local = xbuf + (offset >> 2);
      const uint32_t remote = map_to_rank(smem_u32(xbuf), (uint32_t)owner) + offset;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (c0 >= M) break;
        float v[16];
        // (the whole warp reads tensor memory together: the owners differ from lane to lane only below)
        tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        if (owner == rank) {
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<float4*>(local + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            st_cluster_v4(remote + (uint32_t)((c0 + j) * 4), v[j], v[j + 1], v[j + 2], v[j + 3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  STAMP(6);
  if (S > 1) cluster_sync_all();                 // every slice has arrived at its owner (release / acquire)
  STAMP(7);
  if (warp >= 2 && !abort_flag && !direct) {
    // ---- epilogue of the rows this CTA owns: partial slices added in rank order.  Thread t takes
    // token c = t mod 2^lg (2^lg >= M) and the rows t / 2^lg, + 128 / 2^lg, ...: no division.
    const int et = threadIdx.x - 64;
    const int H = p.mode == D_SWIGLU ? 2 : 1;
    const int half_rows = BM / H;
    const int rows_per = (half_rows + S - 1) / S;
    const int rows_mine = max(0, min(rows_per, half_rows - rank * rows_per));
    const int lg = M <= 1 ? 0 : (M <= 2 ? 1 : (M <= 4 ? 2 : (M <= 8 ? 3 : (M <= 16 ? 4 : (M <= 32 ? 5 : 6)))));
    const int c = et & ((1 << lg) - 1), r0 = et >> lg, rstep = 128 >> lg;
    const int slice = rows_per * BN;             // floats between the slices of two ranks (and halves)
    float ssq = 0.f;
    if (c < M) {
      int it = 0;
      for (int r = r0; r < rows_mine; r += rstep, ++it) {
        const int lrow = rank * rows_per + r;
        const float* src = xbuf + r * BN + c;
        float acc0 = 0.f, acc1 = 0.f;
        if (H == 1) {
          for (int s = 0; s < S; ++s) acc0 += src[s * slice];
        } else {
          for (int s = 0; s < S; ++s) {
            acc0 += src[(2 * s) * slice];
            acc1 += src[(2 * s + 1) * slice];
          }
        }
        if (p.mode == D_SWIGLU) {
          const int ng = n0 + lrow, nu = ng + 64;
          if (nu < N) {
            const float g = acc0 + (p.bias ? p.bias[ng] : 0.f), u = acc1 + (p.bias ? p.bias[nu] : 0.f);
            ((bf16*)p.out)[(size_t)c * p.ldo + (n0 >> 1) + lrow] = __float2bfloat16_rn(silu_mul(g, u));
          }
        } else {
          const int n = n0 + lrow;
          if (n < N) {
            const float val = acc0 + (p.bias ? p.bias[n] : 0.f);
            if (p.mode == D_BF16) {
              ((bf16*)p.out)[(size_t)c * p.ldo + n] = __float2bfloat16_rn(val);
            } else if (p.mode == D_F32) {
              ((float*)p.out)[(size_t)c * p.ldo + n] = val;
            } else {
              float* o = (float*)p.out + (size_t)c * p.ldo + n;
              const float x = (it == 0 ? old_x[0] : (it == 1 ? old_x[1] : __ldcg(o))) + val;
              *o = x;
              ssq += x * x;                      // this thread's rows, in row order
            }
          }
        }
      }
    }
    if (p.mode == D_RESIDUAL && p.ssq_out != nullptr) {
      // partial sums of squares of the new rows over this CTA's columns: the threads of one token
      // are 2^lg apart; a fixed tree inside the warp, then the four warps in order
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        if (o >= (1 << lg)) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
      float* red = xbuf + XBUF_ROWS * BN - 4 * 64;       // the end of the exchange buffer is free (4 warps x 64 tokens)
      if (lg >= 5) {
        // 32 or 64 tokens: a warp holds one or half a row of tokens, nothing to add inside it
        producer_barrier();
        red[(warp - 2) * 64 + c] = ssq;
        producer_barrier();
        if (et < M) {
          float t = 0.f;
          if (lg == 5) { for (int w4 = 0; w4 < 4; ++w4) t += red[w4 * 64 + et]; }
          else { t = red[(et >> 5) * 64 + et] + red[((et >> 5) + 2) * 64 + et]; }
          p.ssq_out[(size_t)(blockIdx.x * S + rank) * p.ssq_out_ld + et] = t;
        }
      } else {
        producer_barrier();                      // everybody has read the slices before their memory is reused
        if (lane < (1 << lg)) red[(warp - 2) * 64 + lane] = ssq;
        producer_barrier();
        if (et < M) {
          const float t = ((red[et] + red[64 + et]) + red[128 + et]) + red[192 + et];
          p.ssq_out[(size_t)(blockIdx.x * S + rank) * p.ssq_out_ld + et] = t;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // copies still in flight may land before the memory goes
  }
  __syncthreads();
  STAMP(8);
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
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
std::unordered_map<WKey, CUtensorMap, WKeyHash> g_wmaps;

int pick_bn(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

// GIBBS_B200_DECODE_XN_KB: the most k-blocks of one CTA whose normalised operand stays in shared
// memory (for comparison runs; at most XN_MAX_KB).
int xn_max_kb() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("GIBBS_B200_DECODE_XN_KB");
    v = e ? atoi(e) : XN_MAX_KB;
    if (v < 1 || v > XN_MAX_KB) v = XN_MAX_KB;
  }
  return v;
}

// How many CTAs share the K of one tile: enough to occupy the SMs, at least four k-blocks each; with
// the norm inside (xn), at least so many that a CTA's operand tiles fit its shared memory.
void plan(int N, int K, bool xn, int* splits, int* kb_per_split) {
  const int total_kb = gb_div_up(K, BK);
  const int tiles = gb_div_up(N, BM);
  int s = 148 / tiles;
  if (s > total_kb / 4) s = total_kb / 4;
  if (xn && s < gb_div_up(total_kb, xn_max_kb())) s = gb_div_up(total_kb, xn_max_kb());
  if (s > MAX_CLUSTER) s = MAX_CLUSTER;
  if (s < 1) s = 1;
  *kb_per_split = gb_div_up(total_kb, s);
  *splits = gb_div_up(total_kb, *kb_per_split);      // no rank is left without a k-block
}

template <int BN>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const DecodeParams& p, cudaStream_t stream) {
  static bool attr_set = false;
  constexpr int MAX_SMEM = DCfg<BN>::SMEM_BYTES + (BN == XN_ROWS ? XN_MAX_KB * XN_TILE_BYTES : 0);
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(gemm_tc_decode_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM));
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(gb_div_up(p.N, BM), 1, p.splits);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = DCfg<BN>::SMEM_BYTES + (p.x_mode ? p.kb_per_split * XN_TILE_BYTES : 0);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = p.splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gb_pdl_enabled() ? 2 : 1;
  GB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_decode_kernel<BN>, tw, tx, p));
  return GB_OK;
}

}  // namespace

// 1 if gb_linear_decode takes a product of these sizes (rows up to 64, a weight TMA can address).
GB_API int gb_linear_decode_supported(int M, const void* W, long long ldw, int K) {
  return (M >= 1 && M <= 64 && K > 0 && K % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)W & 15) == 0) ? 1 : 0;
}

// The number of partial sums of squares per row that a RESIDUAL product of these sizes leaves.
GB_API int gb_linear_decode_parts(int N, int K) {
  int splits, kbs;
  plan(N, K, false, &splits, &kbs);
  return gb_div_up(N, BM) * splits;
}

// 1 if a product of these sizes can run the norm of its rows itself (x_mode 1): up to 16 rows, a K
// range per CTA whose operand tiles fit the shared memory, and no more tiles than one wave of CTAs
// (every CTA normalises the rows for itself: with several waves per SM that work is repeated and
// nothing hides it; such a product reads rows that were normalised once).
GB_API int gb_linear_decode_normed_ok(int M, int N, int K) {
  if (M < 1 || M > XN_ROWS || K % 8 != 0 || gb_div_up(N, BM) > 148) return 0;
  int splits, kbs;
  plan(N, K, true, &splits, &kbs);
  return kbs <= XN_MAX_KB ? 1 : 0;
}

// x_mode 0: X bf16 [M, K] (row stride ldx).  x_mode 1: X float32 rows (the residual stream, row
// stride ldx); row m of the product is rmsnorm(X[rows[m] or m, :K]) * gain, its sum of squares taken
// from ssq_in ([ssq_in_parts][ssq_in_ld] partial sums, indexed by the row of X) or, when ssq_in is
// null, from the row itself.
// W: [N, K] bf16 (row stride ldw); bias f32 [N] or null.
// mode 0: out bf16 [M, N]; 1: out f32 [M, N]; 2: out f32 [M, N] += product, and when ssq_out is not
// null ssq_out[(tile * splits + rank) * ssq_out_ld + m] = sum of squares of the new row m over the
// columns that CTA owns (gb_linear_decode_parts(N, K) partial sums per row); 3: SwiGLU, W rows
// alternating in blocks of 64 between gate and up, out bf16 [M, N / 2].
// flags bit 0: read the weights with an evict-first hint.
// Returns the number of kernels launched (1), or a negative error code.
GB_API int gb_linear_decode(const void* X, long long ldx, int x_mode, const float* gain, float eps, const int* rows,
                            const float* ssq_in, int ssq_in_parts, long long ssq_in_ld, const void* W, long long ldw,
                            const float* bias, void* out, int mode, long long ldo, int M, int N, int K,
                            float* ssq_out, long long ssq_out_ld, int flags, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!gb_linear_decode_supported(M, W, ldw, K))
    GB_FAIL(GB_ERR_ARG, "gb_linear_decode: M = %d (1..64), K = %d and the weight's row stride %lld (multiples of 8, "
            "16-byte aligned base) are not taken", M, K, ldw);
  if (mode < D_BF16 || mode > D_SWIGLU) GB_FAIL(GB_ERR_ARG, "gb_linear_decode: output mode %d", mode);
  if (mode == D_SWIGLU && N % 128 != 0)
    GB_FAIL(GB_ERR_ARG, "gb_linear_decode: the SwiGLU epilogue needs 2 * features = %d to be a multiple of 128", N);
  if (x_mode == 0) {
    if (ldx % 8 != 0 || ((uintptr_t)X & 15) != 0)
      GB_FAIL(GB_ERR_ARG, "gb_linear_decode: bfloat16 rows need a stride that is a multiple of 8 (%lld) and a "
              "16-byte aligned base", ldx);
  } else {
    if (gain == nullptr || ldx % 4 != 0 || ((uintptr_t)X & 15) != 0 || ((uintptr_t)gain & 15) != 0)
      GB_FAIL(GB_ERR_ARG, "gb_linear_decode: normalised rows need a gain, a row stride that is a multiple of 4 "
              "(%lld) and 16-byte aligned bases", ldx);
  }
  if (x_mode != 0 && !gb_linear_decode_normed_ok(M, N, K))
    GB_FAIL(GB_ERR_ARG, "gb_linear_decode: a product of %d rows with K = %d cannot run the norm itself (up to %d rows, "
            "up to %d columns of K per CTA)", M, K, XN_ROWS, XN_MAX_KB * BK);
  const int bn = pick_bn(M);
  DecodeParams p;
  plan(N, K, x_mode != 0, &p.splits, &p.kb_per_split);
  p.total_kb = gb_div_up(K, BK);
  p.x_mode = x_mode;
  p.xn = (const float*)X; p.ldxn = ldx; p.gain = gain; p.eps = eps; p.rows = rows;
  p.ssq_in = ssq_in; p.ssq_in_parts = ssq_in_parts; p.ssq_in_ld = ssq_in_ld; p.K = K;
  p.bias = bias; p.out = out; p.ldo = ldo; p.mode = mode; p.M = M; p.N = N;
  p.ssq_out = ssq_out; p.ssq_out_ld = ssq_out_ld;
  p.stream_weights = (flags & 1) ? 1 : 0;
  p.status = status;

  CUtensorMap tw, tx;
  {
    std::lock_guard<std::mutex> lock(g_wmap_mutex);
    WKey key{W, N, K, ldw};
    auto it = g_wmaps.find(key);
    if (it == g_wmaps.end()) {
      if (!make_tmap(&tw, W, N, K, ldw, BM)) GB_FAIL(GB_ERR_CUDA, "gb_linear_decode: cuTensorMapEncodeTiled failed (W)");
      g_wmaps.emplace(key, tw);
    } else {
      tw = it->second;
    }
  }
  if (x_mode == 0) {
    if (!make_tmap(&tx, X, M, K, ldx, bn)) GB_FAIL(GB_ERR_CUDA, "gb_linear_decode: cuTensorMapEncodeTiled failed (X)");
  } else {
    tx = tw;      // not read
  }
  int rc;
  switch (bn) {
    case 16: rc = launch<16>(tw, tx, p, stream); break;
    case 32: rc = launch<32>(tw, tx, p, stream); break;
    default: rc = launch<64>(tw, tx, p, stream); break;
  }
  if (rc != GB_OK) return rc;
  GB_CHECK_LAUNCH("gb_linear_decode");
  return 1;
}

#ifdef GB_DECODE_TRACE
// Debug builds: where the kernels write their time stamps ([4096][3][16] 64-bit words), or null.
GB_API int gb_linear_decode_trace(unsigned long long* buffer) {
  unsigned int zero = 0;
  GB_CUDA(cudaMemcpyToSymbol(g_trace, &buffer, sizeof(buffer)));
  GB_CUDA(cudaMemcpyToSymbol(g_trace_launch, &zero, sizeof(zero)));
  return GB_OK;
}
#endif

GB_API void gb_linear_decode_forget() {
  std::lock_guard<std::mutex> lock(g_wmap_mutex);
  g_wmaps.clear();
}
