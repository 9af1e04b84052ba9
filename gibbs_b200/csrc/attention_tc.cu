// Causal grouped-query attention over the paged cache in bfloat16 on the
// tensor cores, for a ragged batch: prompt portions and single decoded
// tokens, each request reading its own pages through its block table.
//
// The rows of a CTA's tile are (token, query head of one kv group) pairs, so
// the keys and values of a kv head are read from the pages once for all the
// query heads that share them.  A CTA walks the visible keys in tiles of 64
// absolute positions (cp.async into multi-buffered shared memory, looked up
// page by page), computes S = Q K^T and O += P V with mma.sync m16n8k16, and
// keeps the softmax statistics (running maximum and sum) in 32-bit.
//   prompts: 64 rows per CTA, 16 per warp;  decoding: 16 rows per CTA, the four warps split each tile's keys.
// With splits > 1 (decoding against long contexts) the key range is divided
// among CTAs; each writes an unnormalised partial output with its maximum and
// sum to a workspace and a second kernel merges them in split order.
//
// Formula: MisterTK/gibbs src/graph/cpu.rs:826-951 (keys j <= pos, optional
// window j + w > pos, scale applied to the dot product, max-subtracted
// softmax, query head h reads kv head h / (heads / kv_heads)).
//
// The tensor-core path here is warp-level mma.sync; the matrix products of
// the projections use tcgen05 (gemm_tc.cu).  Attention is 2 % of a prompt's
// arithmetic at these sizes.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

constexpr int KT = 64;   // keys per tile

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (relative error 2^-22; -inf gives 0)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnParams {
  const bf16* q; long long ldq;
  const bf16* k_pages; const bf16* v_pages;
  const int* block_table; int bt_stride; int page_size; int n_pages;
  const int* q_start; const int* q_len; const int* start_pos;
  bf16* out; long long ldo;
  float* part_o; float* part_ml;     // [splits][n_tokens*heads][HD], [splits][n_tokens*heads][2]
  int n_requests, n_tokens, heads, kv_heads, splits, window;
  float scale_log2;                  // scale * log2(e)
  int* status;
};

// Layout of the shared tiles.  Head sizes that are multiples of 64 store rows back to back
// and XOR the 16-byte chunk index with the row (chunk ^ (row & 7)), others pad each row by
// one chunk (an odd number of chunks per row); either way the eight rows an ldmatrix phase
// reads fall in distinct banks.
template <int HD> struct Tile {
  static constexpr int CHUNKS = HD / 8;
  static constexpr bool SWIZZLED = (HD % 64) == 0;
  static constexpr int STRIDE = SWIZZLED ? HD : HD + 8;   // in bf16
  // element offset of (row, col) for col a multiple of 8
  __device__ static __forceinline__ int at(int row, int col) {
    return SWIZZLED ? row * STRIDE + ((((col >> 3) ^ (row & 7)) << 3)) : row * STRIDE + col;
  }
};

// Tiles of keys in flight: prompts double-buffer; decoding CTAs are a single warp that
// waits on memory, so they keep one more tile on the way.
template <bool KSPLIT> struct Depth { static constexpr int STAGES = KSPLIT ? 3 : 2; };

// KSPLIT = false: NW warps, 16 query rows each, every warp walks all 64 keys of a tile.
// KSPLIT = true (decoding): ONE 16-row query tile shared by the NW = 4 warps; warp w takes keys
// 16w .. 16w+15 of every tile with its own running maximum, sum and output, and the four
// partial states are merged through shared memory at the end.  The warps of an SM then have
// something to overlap their memory waits with.
template <int HD, int NW, bool KSPLIT>
__global__ void __launch_bounds__(32 * NW)
attention_tc_kernel(const AttnParams p) {
  pdl_trigger();
  // The wait for the kernel in front (which wrote this step's q, k and v) comes further down: the
  // step's metadata, the page ids and the key tiles that earlier steps filled are fetched first.
  // (Asking L2 for the tiles behind those as well changed nothing: measured, not kept.)
  constexpr int BQ = KSPLIT ? 16 : 16 * NW;
  constexpr int NN = KSPLIT ? 2 : KT / 8;                    // 8-key column tiles per warp and key tile
  using TL = Tile<HD>;
  constexpr int STRIDE = TL::STRIDE, CHUNKS = TL::CHUNKS, NS = Depth<KSPLIT>::STAGES;
  constexpr int NT = 32 * NW;
  extern __shared__ __align__(16) uint8_t smem[];
  bf16* sq = reinterpret_cast<bf16*>(smem);                  // [BQ][STRIDE]
  bf16* sk = sq + BQ * STRIDE;                               // [NS][KT][STRIDE]
  bf16* sv = sk + NS * KT * STRIDE;                          // [NS][KT][STRIDE]
  __shared__ long long row_off[NS + 1][KT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = p.heads / p.kv_heads;
  const int tpt = BQ / group;                                // tokens per tile
  const int kvh = blockIdx.x, z = blockIdx.z;          // x (dispatched fastest) is the kv head: heavy tiles of every head first

  // which request and which of its tiles this CTA has
  // Blocks are handed out in descending order of work: requests from the last to the first and,
  // within a request, from its last tile (which sees the most keys) to its first, so that the
  // long tiles of a causal prompt do not form the tail of the launch.
  int r = p.n_requests - 1, tile = (int)blockIdx.y, found = 0;
  if (KSPLIT) {
    // (a launch of this kind has one tile per request: no search, no dependent loads)
    r -= tile;
    tile = 0;
    found = r >= 0;
  } else {
    for (; r >= 0; --r) {
      const int nt = (p.q_len[r] + tpt - 1) / tpt;
      if (tile < nt) { found = 1; tile = nt - 1 - tile; break; }
      tile -= nt;
    }
  }
  if (!found) return;
  const int qlen = p.q_len[r], first_tok = tile * tpt;
  const int n_tok = min(tpt, qlen - first_tok);             // tokens of this tile
  const int row0 = p.q_start[r] + first_tok;                 // batch row of the tile's first token
  const int pos0 = p.start_pos[r] + first_tok;               // its position
  const int* bt = p.block_table + (size_t)r * p.bt_stride;

  // key range: everything a row of this tile may see, in tiles of KT absolute positions
  const int hi_all = pos0 + n_tok;                           // exclusive
  const int lo_all = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int t_lo = lo_all / KT, t_hi = (hi_all + KT - 1) / KT;
  const int per = (t_hi - t_lo + p.splits - 1) / p.splits;
  const int t_begin = t_lo + z * per, t_end = min(t_hi, t_begin + per);

  const int first_new = p.start_pos[r];                      // positions from here on are written by this step
  // Where each of a tile's 64 keys lies in the pages (element offset of its row, -1: not
  // visible) is worked out once per tile and row, not once per 16-byte piece: slot t % (NS + 1)
  // of row_off belongs to tile t.  It is written an iteration before the tile's loads are
  // issued; the barrier at the head of every iteration makes it visible.
  // The page ids are read early (locate_begin) and turned into offsets late (locate_end), so
  // that the block-table reads of a one-warp CTA overlap the work on the current tile.
  constexpr int RPT = (KT + NT - 1) / NT;                    // rows per thread
  int pending_page[RPT], pending_tile = -1;
  auto locate_begin = [&](int t) {
    pending_tile = t;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int row = tid + i * NT;
      const int j = t * KT + row;
      pending_page[i] = (row < KT && j < hi_all && j >= lo_all) ? bt[j / p.page_size] : -2;   // -2: not visible
    }
  };
  auto locate_end = [&]() {
    if (pending_tile < 0) return;
    const int t = pending_tile;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int row = tid + i * NT;
      if (row >= KT) continue;
      const int j = t * KT + row;
      const int page = pending_page[i];
      long long off = -1;
      if (page >= 0 && page < p.n_pages)
        off = (((long long)page * p.kv_heads + kvh) * p.page_size + j % p.page_size) * HD;
      else if (page != -2)
        atomicExch(p.status, 2);
      row_off[t % (NS + 1)][row] = off;
    }
    pending_tile = -1;
  };
  auto locate = [&](int t) {
    locate_begin(t);
    locate_end();
  };
  auto load_kv = [&](int t, int buf) {
    for (int idx = tid; idx < KT * CHUNKS; idx += NT) {
      const int row = idx / CHUNKS, c = idx - row * CHUNKS;
      const long long off = row_off[t % (NS + 1)][row];
      const bool valid = off >= 0;
      const size_t src = valid ? (size_t)off + c * 8 : 0;
      cp_async_16(sk + buf * KT * STRIDE + TL::at(row, c * 8), p.k_pages + src, valid);
      cp_async_16(sv + buf * KT * STRIDE + TL::at(row, c * 8), p.v_pages + src, valid);
    }
  };
  for (int i = 0; i < NS; ++i)
    if (t_begin + i < t_end) locate(t_begin + i);
  __syncthreads();
  bool waited = false;                     // (the same in every thread of the CTA)
  for (int i = 0; i < NS - 1; ++i) {       // one commit group per tile, also for tiles that do not exist
    if (t_begin + i < t_end) {
      if (!waited && (t_begin + i + 1) * KT > first_new) {
        pdl_wait();
        waited = true;
      }
      load_kv(t_begin + i, i);
    }
    cp_async_commit();
  }
  if (!waited) pdl_wait();
  // Q tile: row = token_local * group + g.  Plain loads (the key tiles above are on their way
  // meanwhile); the barrier at the head of the first iteration makes the tile visible.
  for (int idx = tid; idx < BQ * CHUNKS; idx += NT) {
    const int row = idx / CHUNKS, c = idx - row * CHUNKS;
    const int tl = row / group, g = row - tl * group;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (tl < n_tok)
      v = __ldcg(reinterpret_cast<const uint4*>(p.q + (size_t)(row0 + tl) * p.ldq + (size_t)(kvh * group + g) * HD + c * 8));
    *reinterpret_cast<uint4*>(sq + TL::at(row, c * 8)) = v;
  }

  // this thread's two rows: g0 = lane/4 and g0 + 8 of the warp's 16
  const int wrow = KSPLIT ? 0 : warp * 16;                   // first query row of this warp
  const int kbase = KSPLIT ? warp * 16 : 0;                  // first key (within a tile) of this warp
  const int rloc[2] = {wrow + (lane >> 2), wrow + (lane >> 2) + 8};
  int rpos[2];
  bool rvalid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int tl = rloc[i] / group;
    rvalid[i] = tl < n_tok;
    rpos[i] = pos0 + tl;
  }
  // rows 8..15 of the warp's 16 hold no token when the tile is a decoded token of a group of 8 or fewer
  // heads (then all warps share the rows): their half of the softmax is skipped
  const bool upper = n_tok * group > wrow + 8;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // the maximum in use and the sum under it
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

  uint32_t qf[HD / 16][4];
  for (int t = t_begin; t < t_end; ++t) {
    const int buf = (t - t_begin) % NS;
    cp_async_wait<NS - 2>();               // all but the NS-2 newest groups: tile t (and Q) have landed
    // The one barrier of an iteration: tile t is visible to every warp, every warp has left tile t - 1
    // (whose buffer the next loads overwrite), and the offsets written a tile ago are visible.
    __syncthreads();
    if (t + NS - 1 < t_end) load_kv(t + NS - 1, (t - t_begin + NS - 1) % NS);
    cp_async_commit();
    if (t + NS < t_end) locate_begin(t + NS);      // page ids of a later tile: needed after this tile's work
    if (t == t_begin) {
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk)
        ldmatrix_x4(qf[kk], sq + TL::at(wrow + (lane & 15), kk * 16 + (lane >> 4) * 8));
    }
    // S = Q K^T for this warp's keys of the tile
    float s[NN][4];
#pragma unroll
    for (int n = 0; n < NN; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
    const bf16* kb = sk + buf * KT * STRIDE;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < NN / 2; ++n2) {
        uint32_t b[4];
        ldmatrix_x4(b, kb + TL::at(kbase + n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 16 + ((lane >> 3) & 1) * 8));
        mma_bf16(s[2 * n2], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], qf[kk], b[2], b[3]);
      }
    }
    // scale, mask, the tile's maximum.  A tile that lies below the diagonal (and inside the window) for
    // every row of the CTA needs no mask: rows without a token have q = 0 there, finite and never stored.
    const bool full = t * KT + KT - 1 <= pos0 && (p.window <= 0 || t * KT + p.window > pos0 + n_tok - 1);
    float m_tile[2] = {-INFINITY, -INFINITY};
    if (full) {
#pragma unroll
      for (int n = 0; n < NN; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if ((i >> 1) == 1 && !upper) continue;
          const float v = s[n][i] * p.scale_log2;
          s[n][i] = v;
          m_tile[i >> 1] = fmaxf(m_tile[i >> 1], v);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < NN; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ri = i >> 1;
          if (ri == 1 && !upper) continue;
          const int j = t * KT + kbase + n * 8 + (lane & 3) * 2 + (i & 1);
          const bool vis = rvalid[ri] && j <= rpos[ri] && (p.window <= 0 || j + p.window > rpos[ri]);
          const float v = vis ? s[n][i] * p.scale_log2 : -INFINITY;
          s[n][i] = v;
          m_tile[ri] = fmaxf(m_tile[ri], v);
        }
      }
    }
    // The maximum in use follows the tile's only when it would fall behind by more than 2^8 (P then
    // stays below 256, far inside bfloat16's range); most tiles leave O and the sum as they are.
    float corr[2] = {1.f, 1.f};
#pragma unroll
    for (int ri = 0; ri < 2; ++ri) {
      if (ri == 1 && !upper) continue;
      m_tile[ri] = fmaxf(m_tile[ri], __shfl_xor_sync(0xffffffffu, m_tile[ri], 1));
      m_tile[ri] = fmaxf(m_tile[ri], __shfl_xor_sync(0xffffffffu, m_tile[ri], 2));
      if (m_tile[ri] > m_run[ri] + 8.f || (m_run[ri] == -INFINITY && m_tile[ri] > -INFINITY)) {
        corr[ri] = ex2_approx(m_run[ri] - m_tile[ri]);         // 0 when nothing was seen before
        m_run[ri] = m_tile[ri];
        l_run[ri] *= corr[ri];
      }
    }
    if (corr[0] != 1.f || corr[1] != 1.f) {
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0];
        o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
    }
    // P = exp2(S - m), O += P V
    const bf16* vb = sv + buf * KT * STRIDE;
#pragma unroll
    for (int kk = 0; kk < NN / 2; ++kk) {
      uint32_t a[4];
      float pv[2][4];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ri = i >> 1;
          float e = 0.f;
          if (ri == 0 || upper) {
            e = (m_run[ri] == -INFINITY) ? 0.f : ex2_approx(s[2 * kk + h2][i] - m_run[ri]);
            l_run[ri] += e;
          }
          pv[h2][i] = e;
        }
      a[0] = pack_bf16(pv[0][0], pv[0][1]);
      a[1] = pack_bf16(pv[0][2], pv[0][3]);
      a[2] = pack_bf16(pv[1][0], pv[1][1]);
      a[3] = pack_bf16(pv[1][2], pv[1][3]);
#pragma unroll
      for (int n2 = 0; n2 < HD / 16; ++n2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vb + TL::at(kbase + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, n2 * 16 + (lane >> 4) * 8));
        mma_bf16(o[2 * n2], a, b[0], b[1]);
        mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
      }
    }
    // slot (t + NS) % (NS + 1) held tile t - 1, whose loads were requested an iteration ago; the next
    // iteration's barrier makes these offsets visible before they are used
    locate_end();
  }
  cp_async_wait<0>();

  // row sums across the four threads of a row
#pragma unroll
  for (int ri = 0; ri < 2; ++ri) {
    l_run[ri] += __shfl_xor_sync(0xffffffffu, l_run[ri], 1);
    l_run[ri] += __shfl_xor_sync(0xffffffffu, l_run[ri], 2);
  }
  if constexpr (KSPLIT) {
    // merge the four warps' states: rows 0..15, in warp order
    float* pm = reinterpret_cast<float*>(sk);                // [NW][16] maxima
    float* pl = pm + NW * 16;                                // [NW][16] sums
    float* po = pl + NW * 16;                                // [NW][16][HD] outputs
    const int n_rows = n_tok * group;                        // rows of the tile that hold a (token, head): 16 at most
    __syncthreads();                                         // the key tiles are no longer read
#pragma unroll
    for (int ri = 0; ri < 2; ++ri) {
      const int rr = (lane >> 2) + 8 * ri;
      if (rr >= n_rows) continue;                            // (a decoded token of a group of four fills 4 rows)
      if ((lane & 3) == 0) {
        pm[warp * 16 + rr] = m_run[ri];
        pl[warp * 16 + rr] = l_run[ri];
      }
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<float2*>(po + ((size_t)warp * 16 + rr) * HD + n * 8 + (lane & 3) * 2) =
            make_float2(o[n][2 * ri], o[n][2 * ri + 1]);
    }
    __syncthreads();
    // (only the rows that exist; the warps' weights by the special-function unit, as in the loop above:
    // a decode step waits for these instructions)
    for (int idx = tid; idx < n_rows * HD; idx += NT) {
      const int rr = idx / HD, d = idx - rr * HD;
      const int tl = rr / group, g = rr - tl * group;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) M = fmaxf(M, pm[w * 16 + rr]);
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float mw = pm[w * 16 + rr];
        const float f = (mw == -INFINITY) ? 0.f : ex2_approx(mw - M);
        L += f * pl[w * 16 + rr];
        acc += f * po[((size_t)w * 16 + rr) * HD + d];
      }
      const int trow = row0 + tl, h = kvh * group + g;
      if (p.splits == 1) {
        p.out[(size_t)trow * p.ldo + (size_t)h * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      } else {
        const size_t prow = (size_t)z * p.n_tokens * p.heads + (size_t)trow * p.heads + h;
        p.part_o[prow * HD + d] = acc;
        if (d == 0) {
          p.part_ml[prow * 2] = M;
          p.part_ml[prow * 2 + 1] = L;
        }
      }
    }
    return;
  } else {
#pragma unroll
  for (int ri = 0; ri < 2; ++ri) {
    if (!rvalid[ri]) continue;
    const int tl = rloc[ri] / group, g = rloc[ri] - tl * group;
    const int trow = row0 + tl, h = kvh * group + g;
    if (p.splits == 1) {
      const float inv = l_run[ri] > 0.f ? 1.0f / l_run[ri] : 0.f;
      bf16* dst = p.out + (size_t)trow * p.ldo + (size_t)h * HD + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
            __floats2bfloat162_rn(o[n][2 * ri] * inv, o[n][2 * ri + 1] * inv);
    } else {
      const size_t prow = (size_t)z * p.n_tokens * p.heads + (size_t)trow * p.heads + h;
      float* dst = p.part_o + prow * HD + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * ri], o[n][2 * ri + 1]);
      if ((lane & 3) == 0) {
        p.part_ml[prow * 2] = m_run[ri];
        p.part_ml[prow * 2 + 1] = l_run[ri];
      }
    }
  }
  }
}

// out[row, :] = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z, splits in ascending order.
// One block per row (token, head); at most 32 splits.  The first warp reads all maxima and
// sums at once and leaves the normalised weights in shared memory; then every thread adds
// its column over the splits with the loads of several splits in flight.
__global__ void attention_merge_kernel(const float* part_o, const float* part_ml,
                                       bf16* __restrict__ out, long long ldo, int n_tokens, int heads, int hd,
                                       int splits) {
  __shared__ float wgt[32];
  pdl_trigger();
  const int row = blockIdx.x;                         // token * heads + head
  const size_t rows = (size_t)n_tokens * heads;
  const int t = row / heads, h = row - t * heads;
  // Addresses are worked out (and pinned, see gb_pin) before the wait for the attention kernel;
  // behind it the first instructions are the loads.  Every thread asks for its column of the first
  // sixteen splits before the weights are worked out, so that the outputs and the (maximum, sum)
  // pairs come back in the same trip to L2.
  constexpr int AHEAD = 16;
  const int d_mine = threadIdx.x;
  const float* po = part_o + (size_t)row * hd + (d_mine < hd ? d_mine : 0);
  const float* pml = part_ml + ((size_t)(threadIdx.x < splits ? threadIdx.x : 0) * rows + row) * 2;
  bf16* o = out + (size_t)t * ldo + (size_t)h * hd;
  long long zstride = (long long)(rows * hd);
  gb_pin(po);
  gb_pin(pml);
  gb_pin(o);
  gb_pin(zstride);
  pdl_wait();
  float a[AHEAD];
#pragma unroll
  for (int z = 0; z < AHEAD; ++z) {
    const int zz = z < splits ? z : splits - 1;       // (past the last split: read again, not used)
    a[z] = ldcg_now(po + (size_t)zz * zstride);
  }
  if (threadIdx.x < 32) {
    const int z = threadIdx.x;
    float m = ldcg_now(pml), l = ldcg_now(pml + 1);
    if (z >= splits) {
      m = -INFINITY;
      l = 0.f;
    }
    const float M = warp_max(m);
    const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float L = warp_sum(f * l);
    wgt[z] = L > 0.f ? f / L : 0.f;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    int z = 0;
    if (d == d_mine) {
#pragma unroll
      for (int u = 0; u < AHEAD; ++u)
        if (u < splits) acc += wgt[u] * a[u];
      z = splits < AHEAD ? splits : AHEAD;
    }
    for (; z < splits; ++z) acc += wgt[z] * ldcg_now(part_o + ((size_t)z * rows + row) * hd + d);
    o[d] = __float2bfloat16_rn(acc);
  }
}

template <int HD, bool KSPLIT>
int launch(const AttnParams& p, int n_tiles, cudaStream_t stream) {
  constexpr int NW = 4;
  constexpr int smem = ((KSPLIT ? 16 : 64) + 2 * Depth<KSPLIT>::STAGES * KT) * Tile<HD>::STRIDE * 2;
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    GB_CUDA(cudaFuncSetAttribute(attention_tc_kernel<HD, NW, KSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem));
    attr_set = true;
  }
  dim3 grid(p.kv_heads, n_tiles, p.splits);
  gb_launch(attention_tc_kernel<HD, NW, KSPLIT>, dim3(grid), dim3(32 * NW), smem, stream, p);
  return GB_OK;
}

template <bool KSPLIT>
int dispatch_hd(const AttnParams& p, int hd, int n_tiles, cudaStream_t stream) {
  switch (hd) {
    case 16: return launch<16, KSPLIT>(p, n_tiles, stream);
    case 32: return launch<32, KSPLIT>(p, n_tiles, stream);
    case 48: return launch<48, KSPLIT>(p, n_tiles, stream);
    case 64: return launch<64, KSPLIT>(p, n_tiles, stream);
    case 80: return launch<80, KSPLIT>(p, n_tiles, stream);
    case 96: return launch<96, KSPLIT>(p, n_tiles, stream);
    case 112: return launch<112, KSPLIT>(p, n_tiles, stream);
    case 128: return launch<128, KSPLIT>(p, n_tiles, stream);
  }
  GB_FAIL(GB_ERR_ARG, "gb_attention_tc: head_dim %d is not one of 16, 32, ..., 128", hd);
}

}  // namespace

// 1 if gb_attention_tc takes this geometry.
GB_API int gb_attention_tc_supported(int heads, int kv_heads, int hd, long long ldq, long long ldo) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
  if (hd % 16 != 0 || hd < 16 || hd > 128) return 0;
  if (heads / kv_heads > 64) return 0;
  if (ldq % 8 != 0 || ldo % 2 != 0) return 0;
  return 1;
}

// Number of 32-bit words of workspace for `splits` (0 when splits == 1).
GB_API long long gb_attention_tc_workspace(int n_tokens, int heads, int hd, int splits) {
  return splits > 1 ? (long long)splits * n_tokens * heads * (hd + 2) : 0;
}

// q: [n_tokens, heads*hd] bf16 with row stride ldq (16-byte aligned rows); out likewise with ldo.
// max_q_len: the longest q_len of the batch (known on the host); it selects the tile height.
// Returns the number of kernels launched, or a negative error code.
GB_API int gb_attention_tc(const void* q, long long ldq, const void* k_pages, const void* v_pages,
                           const int* block_table, int bt_stride, int page_size, int n_pages, const int* q_start,
                           const int* q_len, const int* start_pos, void* out, long long ldo, int n_requests,
                           int n_tokens, int max_q_len, int heads, int kv_heads, int hd, float scale, int window,
                           int splits, float* workspace, int* status, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return 0;
  if (!gb_attention_tc_supported(heads, kv_heads, hd, ldq, ldo))
    GB_FAIL(GB_ERR_ARG, "gb_attention_tc: %d heads / %d kv heads / head_dim %d (row strides %lld, %lld) not taken",
            heads, kv_heads, hd, ldq, ldo);
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
    GB_FAIL(GB_ERR_ARG, "gb_attention_tc: q and the pages must be 16-byte aligned");
  if (splits < 1) splits = 1;
  if (splits > 32) GB_FAIL(GB_ERR_ARG, "gb_attention_tc: at most 32 splits, got %d", splits);
  if (splits > 1 && workspace == nullptr) GB_FAIL(GB_ERR_ARG, "gb_attention_tc: splits need a workspace");
  const int group = heads / kv_heads;
  const bool small = (long long)max_q_len * group <= 16 && group <= 16;
  const int bq = small ? 16 : 64;
  if (group > bq) GB_FAIL(GB_ERR_ARG, "gb_attention_tc: %d query heads per kv head", group);
  const int tpt = bq / group;
  // upper bound of the number of tiles: sum_r ceil(q_len_r / tpt) <= n_tokens / tpt + n_requests
  const long long n_tiles = small ? n_requests : ((long long)n_tokens + tpt - 1) / tpt + n_requests;
  if (!small) splits = 1;
  if (n_tiles > 65535) GB_FAIL(GB_ERR_ARG, "gb_attention_tc: %lld tiles in one launch", n_tiles);
  AttnParams p;
  p.q = (const bf16*)q; p.ldq = ldq; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
  p.block_table = block_table; p.bt_stride = bt_stride; p.page_size = page_size; p.n_pages = n_pages;
  p.q_start = q_start; p.q_len = q_len; p.start_pos = start_pos; p.out = (bf16*)out; p.ldo = ldo;
  p.part_o = workspace;
  p.part_ml = workspace ? workspace + (size_t)splits * n_tokens * heads * hd : nullptr;
  p.n_requests = n_requests; p.n_tokens = n_tokens; p.heads = heads; p.kv_heads = kv_heads; p.splits = splits;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  int rc = small ? dispatch_hd<true>(p, hd, (int)n_tiles, stream) : dispatch_hd<false>(p, hd, (int)n_tiles, stream);
  if (rc != GB_OK) return rc;
  GB_CHECK_LAUNCH("gb_attention_tc");
  if (splits > 1) {
    gb_launch(attention_merge_kernel, dim3(n_tokens * heads), dim3(hd <= 64 ? 64 : 128), 0, stream, p.part_o, p.part_ml, (bf16*)out, ldo, n_tokens, heads, hd, splits);
    GB_CHECK_LAUNCH("gb_attention_tc (merge)");
    return 2;
  }
  return 1;
}

