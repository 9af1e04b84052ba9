// Causal grouped-query attention of prompt portions over the paged cache on the 5th generation
// tensor cores: S = Q K^T and O += P V are tcgen05.mma with the accumulators in tensor memory,
// Q, K and V tiles arrive by TMA (K and V page by page through the request's block table), and
// the softmax runs on four warps that own one row each.
//
// A CTA takes one (request, tile of tokens, kv head).  Its 128 rows are (token, query head of the
// kv head's group) pairs, 128 / group tokens, so the keys and values are read once for all the
// heads that share them.  It walks the visible keys in tiles of KEYS = 128 (or 64):
//
//   producer warp   TMA: Q once; then K_j, V_j, K_j+1, ... through a ring of three buffers
//   MMA warp        S = Q K_j^T (tensor memory columns 0..KEYS-1); when the softmax warps have
//                   written P_j: O += P_j V_j (columns KEYS..)
//   softmax warps   thread = row: read S, scale, mask, running maximum m and sum l in 32-bit,
//                   P = exp2(S - m) as bfloat16 into shared memory (the A operand of the second
//                   product); when the maximum has grown by more than 8 (a factor of 256) the
//                   row's O in tensor memory and l are rescaled first; at the end O / l is stored
//
// Two CTAs fit on an SM (97 KB of shared memory and 256 tensor-memory columns each at head_dim
// 64, and at head_dim 128 with 64-key tiles): while one is in its softmax the other's products
// run.  The softmax warps meet at no barrier: each waits for the products itself.
//
// V lies in shared memory as [key][head_dim]: for O = P V it is the B operand with its N index
// contiguous ("MN-major"), which tcgen05 reads directly; nothing is transposed.
//
// Formula: MisterTK/gibbs src/graph/cpu.rs:826-951 (keys j <= pos, optional window j + w > pos,
// scale on the dot product, max-subtracted softmax, query head h reads kv head h / group).
//
// Taken: bfloat16, head_dim 64 or 128, groups of 1 to 16 query heads, page sizes 8..128 that divide 128.
// Every wait is bounded; a wait that runs out sets *status and the CTA drains and returns.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int ROWS = 128;            // rows of a CTA's tile: tokens x heads of the group
constexpr int RING = 3;              // buffers of one K or V tile each
constexpr int STATUS_ATTN_TIMEOUT = 24;

struct Params {
  const int* block_table; int bt_stride; int page_size; int n_pages;
  const int* q_start; const int* q_len; const int* start_pos;
  bf16* out; long long ldo;
  int n_requests, heads, kv_heads, window;
  float scale_log2;
  int* status;
};

// KEYS: keys per tile, 64 or 128.
template <int HD, int KEYS> struct Cfg {
  static constexpr int SUB = HD / 64;                          // 64-column sub-tiles of a K, V or Q tile
  static constexpr int Q_BYTES = ROWS * HD * 2;
  static constexpr int KV_BYTES = KEYS * HD * 2;
  static constexpr int P_BYTES = ROWS * KEYS * 2;
  static constexpr int SMEM_BYTES = Q_BYTES + P_BYTES + RING * KV_BYTES + 1024;
  static constexpr int TMEM_COLS = KEYS + HD <= 128 ? 128 : 256;   // S: KEYS columns, O: HD columns
  // CTAs per SM: by tensor memory (512 columns), shared memory and registers (64 K for 192 threads each).
  // (Three CTAs of 64-key tiles at head_dim 64 were measured: not faster than two.)
  static constexpr int CTAS = SMEM_BYTES <= 113 * 1024 ? 2 : 1;
  static constexpr int REGS = CTAS == 2 ? 168 : 255;
};

// Two 32-bit floats in one 64-bit register: fma / add / sub.f32x2 do two operations in one issue slot.
__device__ __forceinline__ uint64_t pk2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t r, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(r)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// P = exp2(v * scale + neg_m) for one row of a tile, as bfloat16 pairs; returns the row's sum.
template <int KEYS>
__device__ __forceinline__ float exp_row(const float (&v)[KEYS], float scale, float neg_m, uint32_t (&packed)[KEYS / 2]) {
  const uint64_t scale2 = pk2(scale, scale), negm2 = pk2(neg_m, neg_m);
  uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
  for (int i = 0; i < KEYS; i += 2) {
    const int q = i >> 1;
    float x0, x1, e0, e1;
    upk2(fma2(pk2(v[i], v[i + 1]), scale2, negm2), x0, x1);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(x0));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(x1));
    ls2[q & 3] = add2(ls2[q & 3], pk2(e0, e1));
    __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
    packed[q] = *reinterpret_cast<uint32_t*>(&b2);
  }
  float a0, a1, b0, b1;
  upk2(add2(ls2[0], ls2[1]), a0, a1);
  upk2(add2(ls2[2], ls2[3]), b0, b1);
  return (a0 + a1) + (b0 + b1);
}

template <int HD, int KEYS>
__global__ void __launch_bounds__(192) __maxnreg__((Cfg<HD, KEYS>::REGS))
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const Params p) {
  pdl_trigger();
  using C = Cfg<HD, KEYS>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full, kv_full[RING], kv_empty[RING], s_full, s_free, p_full, o_full;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sq = base;                                          // [SUB][128 rows][128 B]
  uint8_t* sp = sq + C::Q_BYTES;                               // [KEYS / 64][128 rows][128 B]: keys 0..63, 64..127
  uint8_t* skv = sp + C::P_BYTES;                              // [RING][SUB][128 keys][128 B]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.heads / p.kv_heads;
  const int tpt = ROWS / group;                                // tokens per tile
  // Blocks are dispatched with x fastest: x is the kv head and y the tile, so that the heavy
  // tiles of every head start first.
  const int kvh = blockIdx.x;

  // Which request and which of its tiles: heaviest first (last request, last tile first).  The
  // three numbers of a request are asked for together, and the barriers are set up while the first
  // request's are on their way: a CTA's start is a chain of trips to memory (these numbers, the
  // block table, the first tiles), and a quarter of all CTA time at 2,048 tokens.
  int r = p.n_requests - 1, tile = (int)blockIdx.y, found = 0;
  int qlen = p.q_len[r], qstart = p.q_start[r], spos = p.start_pos[r];
  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&s_free, 4);                                     // one arrival per softmax warp
    mbar_init(&p_full, 4);                                     // one arrival per softmax warp
    mbar_init(&o_full, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  for (;;) {
    const int nt = (qlen + tpt - 1) / tpt;
    if (tile < nt) { found = 1; tile = nt - 1 - tile; break; }
    tile -= nt;
    if (--r < 0) break;
    qlen = p.q_len[r], qstart = p.q_start[r], spos = p.start_pos[r];
  }
  if (!found) return;
  const int first_tok = tile * tpt;
  const int n_tok = min(tpt, qlen - first_tok);
  const int row0 = qstart + first_tok;                         // batch row of the tile's first token
  const int pos0 = spos + first_tok;                           // its position
  const int hi_all = pos0 + n_tok;                             // keys < hi_all may be visible
  const int lo_all = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int t_lo = lo_all / KEYS, t_hi = (hi_all + KEYS - 1) / KEYS;
  const int n_tiles = t_hi - t_lo;

  if (warp == 1) {
    tmem_alloc(&tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  // The producer's first page ids (the block table is part of the step's metadata, in place before
  // the step's first kernel): asked for here, so that they arrive while the CTA sets up.
  const int* bt = p.block_table + (size_t)r * p.bt_stride;
  const int pages_per_tile = KEYS / p.page_size;
  constexpr int OUTSIDE = -0x7fffffff;
  auto lookup = [&](int t) {
    if (lane >= pages_per_tile) return OUTSIDE;
    const int j0 = t * KEYS + lane * p.page_size;              // first key of this page slot
    return (j0 < hi_all && j0 + p.page_size > lo_all) ? bt[j0 / p.page_size] : OUTSIDE;
  };
  int first_page = 0, page_cur = OUTSIDE;
  if (warp == 0) {
    first_page = bt[lo_all / p.page_size];
    page_cur = t_lo < t_hi ? lookup(t_lo) : OUTSIDE;
    gb_pin(first_page);                                        // (stay in front of the waits below, see gb_pin)
    gb_pin(page_cur);
  }
  if (group * tpt < ROWS) {
    // A group that does not divide 128 (3, 5, 6, 7, ...) leaves the tile's last rows without a
    // (token, head): the q box does not reach them.  They are zeroed so that the tensor core reads
    // numbers there; nothing of these rows is stored.
    const int spare = ROWS - group * tpt;                      // < group <= 16 rows of 128 bytes per sub-tile
    for (int i = threadIdx.x; i < C::SUB * spare * 8; i += blockDim.x) {
      const int sub = i / (spare * 8), rest = i - sub * spare * 8;
      *reinterpret_cast<uint4*>(sq + (size_t)sub * ROWS * 128 + (size_t)(group * tpt + rest / 8) * 128 + (rest & 7) * 16) =
          make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + KEYS;

  if (warp == 0) {
    // ---- producer ----
    pdl_wait();                                                // q and the pages are written by the kernels before
    if (lane == 0) {
      mbar_arrive_expect_tx(&q_full, (uint32_t)(C::SUB * group * tpt * 128));   // the box: tpt tokens x group heads
      for (int sub = 0; sub < C::SUB; ++sub)
        tma_load_3d(sq + (size_t)sub * ROWS * 128, &map_q, sub * 64, kvh * group, row0, &q_full);
    }
    const int page_bytes = p.page_size * 128;                  // of one 64-column sub-tile
    // Lane i brings page slot i of every tile (at most 16 slots).  Its page id for the next tile is
    // read from the block table while this tile's copies are requested, and serves K and V alike: the
    // table is not read between a buffer falling free and its copy going out.
    int it = 0;
    for (int t = t_lo; t < t_hi && !abort_flag; ++t) {
      const int page_next = t + 1 < t_hi ? lookup(t + 1) : OUTSIDE;
      // Slots past the visible range still get data (the products read the whole buffer); any
      // page of the request will do, the mask gives those keys a weight of exactly zero.
      int page = page_cur == OUTSIDE ? first_page : page_cur;
      if (page < 0 || page >= p.n_pages) {
        if (lane < pages_per_tile) atomicExch(p.status, 2);
        page = 0;
      }
      const int row = (page * p.kv_heads + kvh) * p.page_size;
      for (int kv = 0; kv < 2; ++kv, ++it) {                   // K_t, then V_t
        const int s = it % RING;
        bool ok = true;
        if (lane == 0) {
          ok = mbar_wait(&kv_empty[s], ((it / RING) & 1) ^ 1);
          if (!ok) {
            abort_flag = 1;
            atomicExch(p.status, STATUS_ATTN_TIMEOUT);
          } else {
            mbar_arrive_expect_tx(&kv_full[s], C::KV_BYTES);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        uint8_t* dst = skv + (size_t)s * C::KV_BYTES;
        if (lane < pages_per_tile) {
          for (int sub = 0; sub < C::SUB; ++sub)
            tma_load_2d(dst + (size_t)sub * KEYS * 128 + (size_t)lane * page_bytes, kv == 0 ? &map_k : &map_v, sub * 64,
                        row, &kv_full[s]);
        }
      }
      page_cur = page_next;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc_s = idesc_bf16_f32(ROWS, KEYS);
      constexpr uint32_t idesc_o = idesc_bf16_f32_b_mn(ROWS, HD);
      bool ok = mbar_wait(&q_full, 0);
      // Order in the tensor pipe: S_0, then for every tile S_{j+1} before O += P_j V_j.  The softmax
      // warps keep the row of S_j in registers, so S_{j+1} may overwrite it as soon as they have read
      // it (s_free) and is ready when they come back from writing P_j: the products stay out of the
      // softmax warps' way, which set the pace.  Ring items are K_j = 2j and V_j = 2j + 1.
      auto issue_s = [&](int j) {
        const int item = 2 * j, s = item % RING;
        if (!mbar_wait(&kv_full[s], (item / RING) & 1)) return false;
        tc_fence_after();
        const uint8_t* kt = skv + (size_t)s * C::KV_BYTES;
#pragma unroll
        for (int sub = 0; sub < C::SUB; ++sub) {
          const uint64_t da = smem_desc_sw128(sq + (size_t)sub * ROWS * 128);
          const uint64_t db = smem_desc_sw128(kt + (size_t)sub * KEYS * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_s, da + 2 * k, db + 2 * k, idesc_s, (uint32_t)((sub | k) != 0));
        }
        umma_commit(&kv_empty[s]);
        umma_commit(&s_full);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok && !abort_flag; ++j) {
        if (j + 1 < n_tiles) {
          ok = mbar_wait(&s_free, j & 1);
          if (!ok) break;
          tc_fence_after();
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        // O += P V
        {
          const int item = 2 * j + 1, s = item % RING;
          ok = mbar_wait(&p_full, j & 1) && mbar_wait(&kv_full[s], (item / RING) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint8_t* vt = skv + (size_t)s * C::KV_BYTES;
#pragma unroll
          for (int half = 0; half < KEYS / 64; ++half) {       // keys 0..63 (and 64..127) of the tile
            const uint64_t da = smem_desc_sw128(sp + (size_t)half * ROWS * 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              // 16 keys = two 8-row groups of 1024 bytes further in V; a second 64-column block of
              // head_dim (HD = 128) lies one sub-tile further, which the descriptor's leading offset says
              const int key0 = half * 64 + k * 16;
              uint64_t db = smem_desc_sw128(vt + (size_t)key0 * 128);
              if (C::SUB > 1) db = (db & ~((uint64_t)0x3FFF << 16)) | ((uint64_t)((KEYS * 128) >> 4) << 16);
              umma_bf16(tmem_o, da + 2 * k, db, idesc_o, (uint32_t)((j | half | k) != 0));
            }
          }
          umma_commit(&kv_empty[s]);
          umma_commit(&o_full);
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicExch(p.status, STATUS_ATTN_TIMEOUT + 1);
      }
    }
    __syncwarp();
  } else {
    // ---- softmax warps: thread = row ----
    const int q4 = warp & 3;
    const int row = 32 * q4 + lane;
    const int tl = row / group, g = row - tl * group;
    const bool rvalid = tl < n_tok;
    const int rpos = pos0 + tl;
    const uint32_t lane_off = (uint32_t)(32 * q4) << 16;
    float m_used = -INFINITY, l_run = 0.f;
    // A wait that runs out ends this warp's loop (one answer for the whole warp); the other warps
    // see abort_flag at their next tile, or their own waits run out, since this warp no longer arrives.
    bool alive = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int t = t_lo + j;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full, j & 1) && !abort_flag)) {
        abort_flag = 1;
        if (lane == 0) atomicExch(p.status, STATUS_ATTN_TIMEOUT + 2);
        alive = false;
        break;
      }
      tc_fence_after();
      // Which of the tile's columns this row may see: lo_c <= column <= hi_c.  Most tiles lie
      // wholly below the diagonal (and inside the window) for every row: they need no mask.
      const int col0 = t * KEYS;
      const int hi_c = rvalid ? rpos - col0 : -1;
      const int lo_c = (p.window > 0 ? rpos - p.window + 1 : 0) - col0;
      const bool full = col0 + KEYS - 1 <= pos0 && (p.window <= 0 || col0 + p.window > pos0 + tpt - 1);
      const unsigned span = hi_c >= lo_c ? (unsigned)(hi_c - lo_c) : 0u;
      const bool none = hi_c < lo_c;                           // (then `span` is not used)
      // the whole row of S into registers: the loads on their way together, one wait
      float v[KEYS];
#pragma unroll
      for (int c = 0; c < KEYS; c += 32) tmem_ld_32_issue(tmem_s + lane_off + (uint32_t)c, v + c);
      tmem_ld_wait_n<KEYS>(v);
      // the row is in registers: the next tile's first product may overwrite S
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free);
      if (!full) {
#pragma unroll
        for (int i = 0; i < KEYS; ++i) v[i] = (!none && (unsigned)(i - lo_c) <= span) ? v[i] : -INFINITY;
      }
      // the row's maximum over this tile (of the raw products; the scale is positive)
      float mx[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = v[i];
#pragma unroll
      for (int i = 8; i < KEYS; ++i) mx[i & 7] = fmaxf(mx[i & 7], v[i]);
      const float m_tile =
          fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))) *
          p.scale_log2;
      // the maximum in use follows only when it would otherwise fall behind by more than 2^8
      float corr = 1.f;
      const bool grow = m_tile > m_used + 8.f || (m_used == -INFINITY && m_tile > -INFINITY);
      if (grow) {
        corr = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_tile);
        m_used = m_tile;
        l_run *= corr;
      }
      // P = exp2(S * scale - m); a masked column holds -inf and gives exactly 0 (so does every column
      // of a row that has seen nothing yet: -inf * scale + 0 = -inf)
      uint32_t packed[KEYS / 2];
      l_run += exp_row<KEYS>(v, p.scale_log2, (m_used == -INFINITY) ? 0.f : -m_used, packed);
      // P and O of the tile before are still being read by its second product until o_full
      if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(&o_full, (j - 1) & 1))) {
        abort_flag = 1;
        if (lane == 0) atomicExch(p.status, STATUS_ATTN_TIMEOUT + 3);
        alive = false;
        break;
      }
      tc_fence_after();
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          float o[32];
          tmem_ld_32(tmem_o + lane_off + (uint32_t)c0, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= corr;
          tmem_st_32(tmem_o + lane_off + (uint32_t)c0, o);
        }
      }
      // 8 keys (16 bytes) at a time into the swizzled tile
#pragma unroll
      for (int chunk = 0; chunk < KEYS / 8; ++chunk) {
        uint8_t* dst = sp + (size_t)(chunk >> 3) * ROWS * 128 + (size_t)row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) =
            make_uint4(packed[4 * chunk], packed[4 * chunk + 1], packed[4 * chunk + 2], packed[4 * chunk + 3]);
      }
      fence_proxy_async();                                     // P is read by the tensor core (async proxy)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
    }
    if (alive && n_tiles > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(&o_full, (n_tiles - 1) & 1))) {
        abort_flag = 1;
        if (lane == 0) atomicExch(p.status, STATUS_ATTN_TIMEOUT + 4);
        alive = false;
      }
    }
    tc_fence_after();
    if (alive) {
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      bf16* dst = p.out + (size_t)(row0 + tl) * p.ldo + (size_t)(kvh * group + g) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float o[32];
        if (n_tiles > 0) {
          tmem_ld_32(tmem_o + lane_off + (uint32_t)c0, o);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (rvalid) {
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 b2 = __floats2bfloat162_rn(o[c8 * 8 + 2 * e] * inv, o[c8 * 8 + 2 * e + 1] * inv);
              pk[e] = *reinterpret_cast<uint32_t*>(&b2);
            }
            *reinterpret_cast<uint4*>(dst + c0 + c8 * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);          // copies still in flight land before the memory goes
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_slot, C::TMEM_COLS);
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

bool encode(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
            const cuuint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct PagesKey {
  const void* p; long long rows; int hd, page_size;
  bool operator==(const PagesKey& o) const { return p == o.p && rows == o.rows && hd == o.hd && page_size == o.page_size; }
};
struct PagesKeyHash {
  size_t operator()(const PagesKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.rows) * 31) ^ (size_t)(k.hd * 131 + k.page_size);
  }
};
std::mutex g_mutex;
std::unordered_map<PagesKey, CUtensorMap, PagesKeyHash> g_page_maps;   // the pools do not move: their maps are made once

bool pages_map(CUtensorMap* out, const void* pages, long long rows, int hd, int page_size) {
  std::lock_guard<std::mutex> lock(g_mutex);
  PagesKey key{pages, rows, hd, page_size};
  auto it = g_page_maps.find(key);
  if (it != g_page_maps.end()) {
    *out = it->second;
    return true;
  }
  cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  if (!encode(out, pages, 2, dims, strides, box)) return false;
  g_page_maps.emplace(key, *out);
  return true;
}

template <int HD, int KEYS>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, int n_tiles,
           cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    GB_CUDA(cudaFuncSetAttribute(attention_tcgen05_kernel<HD, KEYS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<HD, KEYS>::SMEM_BYTES));
    attr_set = true;
  }
  gb_launch(attention_tcgen05_kernel<HD, KEYS>, dim3(p.kv_heads, n_tiles), dim3(192), Cfg<HD, KEYS>::SMEM_BYTES, stream,
            mq, mk, mv, p);
  return GB_OK;
}

// Keys per tile.  At head_dim 128 a CTA of 128-key tiles has an SM to itself (161 KB of shared
// memory); with 64-key tiles two fit, which is the faster way once the launch has several CTAs for
// every SM (8,192 tokens x 16 / 4 heads: 335 us against 432 us; 4,096: 98 against 125; at 2,048, 260 CTAs, 50
// against 40).  At head_dim 64 two CTAs fit either way and the wider tile is faster (462 us
// against 567 us at 8,192 tokens x 32 / 8 heads).  GIBBS_B200_ATTN_KEYS=64|128 overrides.
int keys_per_tile(int hd, int page_size, long long ctas) {
  static const int forced = [] {
    const char* e = getenv("GIBBS_B200_ATTN_KEYS");
    return e ? atoi(e) : 0;
  }();
  if (page_size > 64) return 128;
  if (forced == 64 || forced == 128) return forced;
  return (hd == 128 && ctas >= 3 * 148) ? 64 : 128;
}

}  // namespace

// 1 if gb_attention_tcgen05 takes this geometry.
GB_API int gb_attention_tcgen05_supported(int heads, int kv_heads, int hd, int page_size, long long ldq, long long ldo) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
  const int group = heads / kv_heads;
  if (group > 16) return 0;
  if (hd != 64 && hd != 128) return 0;
  if (page_size < 8 || page_size > 128 || 128 % page_size != 0) return 0;
  if (ldq % 8 != 0 || ldo % 8 != 0) return 0;
  return 1;
}

// The arguments of gb_attention_tc (attention_tc.cu) without splits: q [n_tokens, heads*hd] bf16 with row
// stride ldq, pages [n_pages, kv_heads, page_size, hd] bf16, out [n_tokens, heads*hd] bf16 with row stride ldo.
// Returns the number of kernels launched, or a negative error code.
GB_API int gb_attention_tcgen05(const void* q, long long ldq, const void* k_pages, const void* v_pages,
                                const int* block_table, int bt_stride, int page_size, int n_pages, const int* q_start,
                                const int* q_len, const int* start_pos, void* out, long long ldo, int n_requests,
                                int n_tokens, int heads, int kv_heads, int hd, float scale, int window, int* status,
                                cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return 0;
  if (!gb_attention_tcgen05_supported(heads, kv_heads, hd, page_size, ldq, ldo))
    GB_FAIL(GB_ERR_ARG, "gb_attention_tcgen05: %d heads / %d kv heads / head_dim %d / pages of %d (row strides %lld, "
            "%lld) not taken", heads, kv_heads, hd, page_size, ldq, ldo);
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 15))
    GB_FAIL(GB_ERR_ARG, "gb_attention_tcgen05: q, out and the pages must be 16-byte aligned");
  if (!(scale > 0.f)) GB_FAIL(GB_ERR_ARG, "gb_attention_tcgen05: the scale must be positive, got %g", (double)scale);
  const int group = heads / kv_heads;
  const int tpt = ROWS / group;
  CUtensorMap mq, mk, mv;
  {
    // q as [token][head][hd]: a box of 64 columns x the group's heads x the tile's tokens lands as rows (token, head)
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)ldq * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)tpt};
    if (!encode(&mq, q, 3, dims, strides, box)) GB_FAIL(GB_ERR_CUDA, "gb_attention_tcgen05: cuTensorMapEncodeTiled failed (q)");
  }
  const long long page_rows = (long long)n_pages * kv_heads * page_size;
  if (!pages_map(&mk, k_pages, page_rows, hd, page_size) || !pages_map(&mv, v_pages, page_rows, hd, page_size))
    GB_FAIL(GB_ERR_CUDA, "gb_attention_tcgen05: cuTensorMapEncodeTiled failed (pages)");
  Params p;
  p.block_table = block_table; p.bt_stride = bt_stride; p.page_size = page_size; p.n_pages = n_pages;
  p.q_start = q_start; p.q_len = q_len; p.start_pos = start_pos; p.out = (bf16*)out; p.ldo = ldo;
  p.n_requests = n_requests; p.heads = heads; p.kv_heads = kv_heads; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  // upper bound of the number of tiles: sum_r ceil(q_len_r / tpt) <= n_tokens / tpt + n_requests
  const long long n_tiles = ((long long)n_tokens + tpt - 1) / tpt + n_requests;
  if (n_tiles > 65535) GB_FAIL(GB_ERR_ARG, "gb_attention_tcgen05: %lld tiles in one launch", n_tiles);
  int rc;
  if (keys_per_tile(hd, page_size, n_tiles * kv_heads) == 64)
    rc = hd == 64 ? launch<64, 64>(mq, mk, mv, p, (int)n_tiles, stream) : launch<128, 64>(mq, mk, mv, p, (int)n_tiles, stream);
  else
    rc = hd == 64 ? launch<64, 128>(mq, mk, mv, p, (int)n_tiles, stream) : launch<128, 128>(mq, mk, mv, p, (int)n_tiles, stream);
  if (rc != GB_OK) return rc;
  GB_CHECK_LAUNCH("gb_attention_tcgen05");
  return 1;
}

// Forget the tensor maps of page pools (an engine that frees its pools calls this).
GB_API void gb_attention_tcgen05_forget() {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_page_maps.clear();
}
