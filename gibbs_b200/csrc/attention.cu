// Attention over the paged cache, for a ragged batch of prompt portions and
// single decoded tokens.
//
//  gb_qk_norm_rope_store: per-head RMSNorm of q and k (optional), rotary
//    position encoding of q and k (optional; half-split or adjacent pairs),
//    q rewritten in place, k and v written into the pages of their positions.
//    The rotary table `inv_freq` holds rotary_dim / 2 frequencies followed by
//    ONE more value, the factor the cosines and sines are multiplied by (the
//    reference's rope mscale, src/graph/cpu.rs:674-675; 1 for LFM2).
//  gb_paged_attention: for every (token, head) softmax((q.K_j)*scale) V_j over
//    the visible keys j <= pos (and j > pos - window), read through the
//    request's block table; with softcap > 0 the scaled scores pass through
//    cap * tanh(s / cap) first (the reference's soft_cap,
//    arch/lib/transformer.json5:69-75).
//
// Formulas (MisterTK/gibbs): per-head norm arch/lib/transformer.json5:22-24,
// 55-58; RoPE src/graph/cpu.rs:632-697 (angle = (float)pos * inv_freq[j] in
// 32-bit); attention src/graph/cpu.rs:826-951 (keys are written first, query
// head h reads kv head h / (heads/kv_heads), max-subtracted softmax).
//
// Page layout: [n_pages, kv_heads, page_size, head_dim]; position p of a
// request lives in page block_table[request][p / page_size] at row
// p % page_size.  A page id outside 0..n_pages-1 is never dereferenced: the
// access is skipped and *status is set to a nonzero code.
#include "common.cuh"

namespace {

enum { STATUS_BAD_PAGE_WRITE = 1, STATUS_BAD_PAGE_READ = 2 };

template <typename T>
__global__ void qk_norm_rope_store_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ q_gain,
                                          const float* __restrict__ k_gain, float eps,
                                          const float* __restrict__ inv_freq, int rotary_dim, int adjacent,
                                          const int* tok_req, const int* tok_pos,
                                          const int* block_table, int bt_stride, int page_size,
                                          T* __restrict__ k_pages, T* __restrict__ v_pages, int n_pages,
                                          int n_tokens, int heads, int kv_heads, int hd, int write_kv,
                                          int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= (long long)n_tokens * slots) return;
  const int t = (int)(idx / slots), slot = (int)(idx - (long long)t * slots);
  const int pos = tok_pos[t];
  // columns of the fused row: [q heads | k heads | v heads]
  T* src = qkv + (size_t)t * ld + (size_t)slot * hd;
  const bool is_q = slot < heads;
  const bool is_k = !is_q && slot < heads + kv_heads;
  const int kvh = is_q ? 0 : (is_k ? slot - heads : slot - heads - kv_heads);

  T* dst = src;  // q in place
  if (!is_q) {
    const int page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
    if (page < 0 || page >= n_pages) {
      if (lane == 0) atomicExch(status, STATUS_BAD_PAGE_WRITE);
      return;
    }
    T* pages = is_k ? k_pages : v_pages;
    dst = pages + (((size_t)page * kv_heads + kvh) * page_size + pos % page_size) * hd;
  }
  if (!is_q && !is_k) {  // v: plain copy
    for (int d = lane; d < hd; d += 32) dst[d] = src[d];
    return;
  }
  const float* gain = is_q ? q_gain : k_gain;
  float scale = 1.f;
  if (gain) {
    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) {
      const float v = to_f32(src[d]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    scale = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  const int half = inv_freq ? rotary_dim / 2 : 0;
  const float mscale = inv_freq ? inv_freq[half] : 1.f;
  for (int j = lane; j < half; j += 32) {
    const int i0 = adjacent ? 2 * j : j;
    const int i1 = adjacent ? 2 * j + 1 : j + half;
    float a = to_f32(src[i0]), b = to_f32(src[i1]);
    if (gain) {
      a = a * scale * gain[i0];
      b = b * scale * gain[i1];
    }
    const float ang = (float)pos * inv_freq[j];
    const float c = cosf(ang) * mscale, s = sinf(ang) * mscale;
    dst[i0] = from_f32<T>(a * c - b * s);
    dst[i1] = from_f32<T>(a * s + b * c);
  }
  for (int d = 2 * half + lane; d < hd; d += 32) {
    float a = to_f32(src[d]);
    if (gain) a = a * scale * gain[d];
    dst[d] = from_f32<T>(a);
  }
}

// Prompt portions in bfloat16 at head sizes 32, 64 and 128 with the half-split rotation over the
// whole head: one block per token.  The token's cosines and sines are worked out once (not once
// per head) into shared memory; then hd/8 threads share a head, each with 8 neighbouring values
// in one 16-byte load, the sum of squares and the rotation partner (hd/2 further) coming from the
// neighbouring threads by shuffles.  Same arithmetic as the kernel above, value by value.
__global__ void qk_norm_rope_store_vec_kernel(bf16* __restrict__ qkv, long long ld, const float* __restrict__ q_gain,
                                              const float* __restrict__ k_gain, float eps,
                                              const float* __restrict__ inv_freq, const int* tok_req,
                                              const int* tok_pos, const int* block_table,
                                              int bt_stride, int page_size, bf16* __restrict__ k_pages,
                                              bf16* __restrict__ v_pages, int n_pages, int heads, int kv_heads, int hd,
                                              int write_kv, int* __restrict__ status) {
  __shared__ float cs[64], sn[64];                       // hd / 2 <= 64
  pdl_trigger();
  const int t = blockIdx.x;
  const int half = hd >> 1;
  const int tps = hd >> 3;                               // threads per head: 4, 8 or 16
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  const int total = slots * tps;                         // a multiple of 4; the block is padded to whole warps
  // Position, page and angles come from the step's metadata and from tables: they are worked out
  // before the wait for the product in front, and this thread's first piece of the row is
  // requested right after it, before anything that would make it wait.
  const int pos = tok_pos[t];
  const float mscale = inv_freq[half];
  int page = 0;
  bool bad_page = false;
  if (write_kv) {
    page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
    bad_page = page < 0 || page >= n_pages;
  }
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const float ang = (float)pos * inv_freq[j];
    cs[j] = cosf(ang) * mscale;
    sn[j] = sinf(ang) * mscale;
  }
  gb_pin(page);                                          // (stays in front of the wait, see gb_pin)
  gb_pin(bad_page);
  pdl_wait();
  uint4 raw0 = make_uint4(0, 0, 0, 0);
  if ((int)threadIdx.x < total) {
    const int slot0 = threadIdx.x / tps, sub0 = threadIdx.x - slot0 * tps;
    raw0 = __ldcg(reinterpret_cast<const uint4*>(qkv + (size_t)t * ld + (size_t)slot0 * hd + sub0 * 8));
  }
  __syncthreads();
  if (bad_page) {
    if (threadIdx.x == 0) atomicExch(status, STATUS_BAD_PAGE_WRITE);
    write_kv = 0;                                        // q is still processed
  }
  for (int idx0 = 0; idx0 < total; idx0 += blockDim.x) {
    const int idx = idx0 + threadIdx.x;
    const bool active = idx < total;
    const int slot = active ? idx / tps : 0, sub = active ? idx - slot * tps : 0;
    const bool is_q = slot < heads;
    const bool is_k = !is_q && slot < heads + kv_heads;
    const int kvh = is_q ? 0 : (is_k ? slot - heads : slot - heads - kv_heads);
    bf16* src = qkv + (size_t)t * ld + (size_t)slot * hd + sub * 8;
    float v[8];
    {
      const uint4 raw = idx0 == 0 ? raw0 : (active ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        v[2 * e] = f.x;
        v[2 * e + 1] = f.y;
      }
    }
    bf16* dst = src;
    if (!is_q) dst = (is_k ? k_pages : v_pages) + (((size_t)page * kv_heads + kvh) * page_size + pos % page_size) * hd + sub * 8;
    const bool store = active && (is_q || write_kv);
    const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);
    // every lane takes part in the shuffles; a head's threads are neighbours within a warp
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    for (int o = tps >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (gain) {
      const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = v[e] * scale * gain[sub * 8 + e];
    }
    float w[8];                                          // the partner's values: hd/2 further (or back)
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = __shfl_xor_sync(0xffffffffu, v[e], tps >> 1);
    if (is_q || is_k) {
      const bool lower = sub < (tps >> 1);
      const int j0 = (lower ? sub : sub - (tps >> 1)) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float c = cs[j0 + e], sv = sn[j0 + e];
        v[e] = lower ? (v[e] * c - w[e] * sv) : (w[e] * sv + v[e] * c);
      }
    }
    if (store) {
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
      *reinterpret_cast<uint4*>(dst) = o;
    }
  }
}

// The same for q, k, v given as the partial tiles of the split-K product that made them
// (ws[split][token][cols], 32-bit, plus bias): the sums are rounded to bfloat16 where the
// product's own reduction would have rounded them.  q goes to q_out [n_tokens, heads*hd].
__global__ void qk_norm_rope_store_partials_kernel(const float* ws, int splits, const float* __restrict__ bias,
                                                   bf16* __restrict__ q_out, const float* __restrict__ q_gain,
                                                   const float* __restrict__ k_gain, float eps,
                                                   const float* __restrict__ inv_freq, int rotary_dim, int adjacent,
                                                   const int* tok_req, const int* tok_pos,
                                                   const int* block_table, int bt_stride, int page_size,
                                                   bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, int n_pages,
                                                   int n_tokens, int heads, int kv_heads, int hd, int write_kv,
                                                   int async_copies, int* __restrict__ status) {
  // per warp: [hd] sums, then (async_copies) [splits][hd] copies of the partial tiles
  extern __shared__ __align__(16) float staged[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_warp = hd * (async_copies ? splits + 1 : 1);
  float* mine = staged + (size_t)warp * per_warp;
  float* parts = mine + hd;
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  const int cols = slots * hd;
  const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (idx >= (long long)n_tokens * slots) return;
  const int t = (int)(idx / slots), slot = (int)(idx - (long long)t * slots);
  // Everything but the product's partial tiles is read, and the rotation worked out, before the
  // wait for the product: position and page from the step's metadata, gains, bias, angles.
  const int pos = tok_pos[t];
  const bool is_q = slot < heads;
  const bool is_k = !is_q && slot < heads + kv_heads;
  const int kvh = is_q ? 0 : (is_k ? slot - heads : slot - heads - kv_heads);
  bf16* dst;
  bool bad_page = false;
  if (is_q) {
    dst = q_out + (size_t)t * heads * hd + (size_t)slot * hd;
  } else {
    const int page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
    bad_page = page < 0 || page >= n_pages;
    dst = (is_k ? k_pages : v_pages) + (((size_t)(bad_page ? 0 : page) * kv_heads + kvh) * page_size + pos % page_size) * hd;
  }
  const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);
  const int half = (inv_freq && (is_q || is_k)) ? rotary_dim / 2 : 0;
  const float mscale = half ? inv_freq[half] : 1.f;
  constexpr int PRE = 2;                                 // rotation pairs per lane prepared ahead (head sizes up to 128)
  float pc[PRE], ps[PRE], pg0[PRE], pg1[PRE];
#pragma unroll
  for (int k = 0; k < PRE; ++k) {
    const int jj = lane + 32 * k;
    pc[k] = 1.f; ps[k] = 0.f; pg0[k] = 1.f; pg1[k] = 1.f;
    if (jj < half) {
      const float ang = (float)pos * inv_freq[jj];
      pc[k] = cosf(ang) * mscale;
      ps[k] = sinf(ang) * mscale;
      if (gain) {
        pg0[k] = gain[adjacent ? 2 * jj : jj];
        pg1[k] = gain[adjacent ? 2 * jj + 1 : jj + half];
      }
    }
  }
  float pb[4] = {0.f, 0.f, 0.f, 0.f};                    // bias of this lane's first four columns
  if (bias) {
#pragma unroll
    for (int m = 0; m < 4; ++m)
      if (lane + 32 * m < hd) pb[m] = bias[slot * hd + lane + 32 * m];
  }
  // (pinned: all of this stays in front of the wait, see gb_pin)
#pragma unroll
  for (int k = 0; k < PRE; ++k) { gb_pin(pc[k]); gb_pin(ps[k]); gb_pin(pg0[k]); gb_pin(pg1[k]); }
#pragma unroll
  for (int m = 0; m < 4; ++m) gb_pin(pb[m]);
  gb_pin(dst);
  gb_pin(bad_page);
  const size_t split_stride = (size_t)n_tokens * cols;
  const float* row0 = ws + (size_t)t * cols + (size_t)slot * hd;
  pdl_wait();
  if (bad_page) {
    if (lane == 0) atomicExch(status, STATUS_BAD_PAGE_WRITE);
    return;
  }
  if (async_copies) {
    // all splits of this head's row in one trip to L2: hd / 4 pieces of 16 bytes per split
    const int pieces = hd >> 2;
    for (int i = lane; i < splits * pieces; i += 32) {
      const int sp = i / pieces, c = i - sp * pieces;
      gb_cp_async_16(parts + (size_t)sp * hd + 4 * c, row0 + (size_t)sp * split_stride + 4 * c);
    }
    gb_cp_async_wait_all();
    __syncwarp();
  }
  float ss = 0.f;
  for (int d0 = 0; d0 < hd; d0 += 128) {                 // four columns per lane at a time
    float v[4];
    if (async_copies) {
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int d = d0 + lane + 32 * m;
        v[m] = 0.f;
        if (d < hd)
          for (int sp = 0; sp < splits; ++sp) v[m] += parts[(size_t)sp * hd + d];
      }
    } else {
      size_t at[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int d = d0 + lane + 32 * m;
        at[m] = (size_t)t * cols + (size_t)slot * hd + (d < hd ? d : hd - 1);
      }
      sum_partials<4>(ws, splits, split_stride, at, v);
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int d = d0 + lane + 32 * m;
      if (d < hd) {
        if (bias) v[m] += d0 == 0 ? pb[m] : bias[slot * hd + d];
        const float x = to_f32(from_f32<bf16>(v[m]));
        mine[d] = x;
        ss += x * x;
      }
    }
  }
  __syncwarp();
  if (!is_q && !is_k) {
    for (int d = lane; d < hd; d += 32) dst[d] = __float2bfloat16_rn(mine[d]);
    return;
  }
  float scale = 1.f;
  if (gain) {
    ss = warp_sum(ss);
    scale = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  for (int j = lane, k = 0; j < half; j += 32, ++k) {
    const int i0 = adjacent ? 2 * j : j;
    const int i1 = adjacent ? 2 * j + 1 : j + half;
    float a = mine[i0], b = mine[i1];
    float c, sn;
    if (k < PRE) {
      // (static indexing keeps the prepared values in registers)
      c = k == 0 ? pc[0] : pc[1];
      sn = k == 0 ? ps[0] : ps[1];
      if (gain) {
        a = a * scale * (k == 0 ? pg0[0] : pg0[1]);
        b = b * scale * (k == 0 ? pg1[0] : pg1[1]);
      }
    } else {
      if (gain) {
        a = a * scale * gain[i0];
        b = b * scale * gain[i1];
      }
      const float ang = (float)pos * inv_freq[j];
      c = cosf(ang) * mscale;
      sn = sinf(ang) * mscale;
    }
    dst[i0] = __float2bfloat16_rn(a * c - b * sn);
    dst[i1] = __float2bfloat16_rn(a * sn + b * c);
  }
  for (int d = 2 * half + lane; d < hd; d += 32) {
    float a = mine[d];
    if (gain) a = a * scale * gain[d];
    dst[d] = __float2bfloat16_rn(a);
  }
}

// One warp per (token, head).  Lane l takes the keys lo + l, lo + l + 32, ...
// with its own running (max, sum, output); the 32 partial states are merged at
// the end.  Which keys a lane takes depends on the query's position only, so
// the result is the same however the batch was cut.
template <typename T, int HD_MAX>
__global__ void __launch_bounds__(128)
paged_attention_kernel(const T* q, long long ldq, const T* k_pages,
                       const T* v_pages, const int* block_table, int bt_stride,
                       int page_size, int n_pages, const int* tok_req,
                       const int* tok_pos, T* __restrict__ out, long long ldo, int n_tokens,
                       int heads, int kv_heads, int hd, float scale, float softcap, int window,
                       int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  __shared__ float qs[4][HD_MAX];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long idx = (long long)blockIdx.x * 4 + warp;
  if (idx >= (long long)n_tokens * heads) return;
  const int t = (int)(idx / heads), h = (int)(idx - (long long)t * heads);
  const int kvh = h / (heads / kv_heads);
  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_req[t] * bt_stride;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = to_f32(q[(size_t)t * ldq + (size_t)h * hd + d]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float o[HD_MAX];
#pragma unroll
  for (int d = 0; d < HD_MAX; ++d) o[d] = 0.f;

  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int j = lo + lane; j <= pos; j += 32) {
    const int page = bt[j / page_size];
    if (page < 0 || page >= n_pages) {
      atomicExch(status, STATUS_BAD_PAGE_READ);
      continue;
    }
    const size_t row = (((size_t)page * kv_heads + kvh) * page_size + j % page_size) * hd;
    const T* kp = k_pages + row;
    const T* vp = v_pages + row;
    float dot = 0.f;
#pragma unroll
    for (int d = 0; d < HD_MAX; ++d)
      if (d < hd) dot = fmaf(qs[warp][d], to_f32(kp[d]), dot);
    float s = dot * scale;
    if (softcap > 0.f) s = softcap * tanhf(s / softcap);       // scores squashed into (-cap, cap)
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float p = expf(s - m_new);
    l = l * corr + p;
#pragma unroll
    for (int d = 0; d < HD_MAX; ++d)
      if (d < hd) o[d] = o[d] * corr + p * to_f32(vp[d]);
    m = m_new;
  }

  const float m_all = warp_max(m);
  const float f = (m == -INFINITY) ? 0.f : expf(m - m_all);
  const float l_all = warp_sum(l * f);
  const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
  T* dst = out + (size_t)t * ldo + (size_t)h * hd;
#pragma unroll
  for (int d = 0; d < HD_MAX; ++d) {
    if (d < hd) {
      const float v = warp_sum(o[d] * f);
      if ((d & 31) == lane) dst[d] = from_f32<T>(v * inv);
    }
  }
}

template <typename T>
int launch_attention(const void* q, long long ldq, const void* k_pages, const void* v_pages, const int* block_table,
                     int bt_stride, int page_size, int n_pages, const int* tok_req, const int* tok_pos, void* out,
                     long long ldo, int n_tokens, int heads, int kv_heads, int hd, float scale, float softcap,
                     int window, int* status, cudaStream_t stream) {
  const long long warps = (long long)n_tokens * heads;
  const int blocks = gb_div_up(warps, 4);
#define GB_ATTN(HD)                                                                                              \
  gb_launch(paged_attention_kernel<T, HD>, dim3(blocks), dim3(128), 0, stream, (const T*)q, ldq, (const T*)k_pages, (const T*)v_pages, \
                                                            block_table, bt_stride, page_size, n_pages, tok_req, \
                                                            tok_pos, (T*)out, ldo, n_tokens, heads, kv_heads, hd, \
                                                            scale, softcap, window, status)
  if (hd <= 32) GB_ATTN(32);
  else if (hd <= 64) GB_ATTN(64);
  else if (hd <= 128) GB_ATTN(128);
  else GB_ATTN(256);
#undef GB_ATTN
  return 0;
}

}  // namespace

GB_API int gb_qk_norm_rope_store(void* qkv, int dtype, long long ld, const float* q_gain, const float* k_gain,
                                 float eps, const float* inv_freq, int rotary_dim, int adjacent, const int* tok_req,
                                 const int* tok_pos, const int* block_table, int bt_stride, int page_size,
                                 void* k_pages, void* v_pages, int n_pages, int n_tokens, int heads, int kv_heads,
                                 int hd, int write_kv, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return GB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0)
    GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store: %d heads over %d kv heads", heads, kv_heads);
  if (inv_freq && (rotary_dim % 2 != 0 || rotary_dim > hd || rotary_dim <= 0))
    GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store: rotary_dim %d for head_dim %d", rotary_dim, hd);
  if (page_size <= 0) GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store: page_size %d", page_size);
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  if (dtype == GB_BF16 && n_tokens >= 32 && (hd == 32 || hd == 64 || hd == 128) && inv_freq != nullptr && !adjacent &&
      rotary_dim == hd && ld % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 &&
      ((uintptr_t)v_pages & 15) == 0) {
    int threads = slots * (hd / 8);
    threads = threads > 512 ? 512 : ((threads + 31) / 32) * 32;
    gb_launch(qk_norm_rope_store_vec_kernel, dim3(n_tokens), dim3(threads), 0, stream, (bf16*)qkv, ld, q_gain, k_gain,
              eps, inv_freq, tok_req, tok_pos, block_table, bt_stride, page_size, (bf16*)k_pages, (bf16*)v_pages,
              n_pages, heads, kv_heads, hd, write_kv, status);
    GB_CHECK_LAUNCH("gb_qk_norm_rope_store (vector)");
    return GB_OK;
  }
  const long long warps = (long long)n_tokens * slots;
  const int blocks = gb_div_up(warps, 4);
  if (dtype == GB_F32)
    gb_launch(qk_norm_rope_store_kernel<float>, dim3(blocks), dim3(128), 0, stream, (float*)qkv, ld, q_gain, k_gain, eps, inv_freq, rotary_dim, adjacent, tok_req, tok_pos, block_table,
        bt_stride, page_size, (float*)k_pages, (float*)v_pages, n_pages, n_tokens, heads, kv_heads, hd, write_kv,
        status);
  else if (dtype == GB_BF16)
    gb_launch(qk_norm_rope_store_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, (bf16*)qkv, ld, q_gain, k_gain, eps, inv_freq, rotary_dim, adjacent, tok_req, tok_pos, block_table,
        bt_stride, page_size, (bf16*)k_pages, (bf16*)v_pages, n_pages, n_tokens, heads, kv_heads, hd, write_kv,
        status);
  else
    GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store: unknown dtype %d", dtype);
  GB_CHECK_LAUNCH("gb_qk_norm_rope_store");
  return GB_OK;
}

// q, k, v as the `splits` partial tiles (32-bit [splits][n_tokens][cols], cols = (heads + 2*kv_heads) * hd,
// or heads * hd without write_kv) of a split-K product, plus its bias or null; bfloat16 pages and q_out.
GB_API int gb_qk_norm_rope_store_partials(const float* ws, int splits, const float* bias, void* q_out,
                                          const float* q_gain, const float* k_gain, float eps, const float* inv_freq,
                                          int rotary_dim, int adjacent, const int* tok_req, const int* tok_pos,
                                          const int* block_table, int bt_stride, int page_size, void* k_pages,
                                          void* v_pages, int n_pages, int n_tokens, int heads, int kv_heads, int hd,
                                          int write_kv, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return GB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0)
    GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store_partials: %d heads over %d kv heads", heads, kv_heads);
  if (inv_freq && (rotary_dim % 2 != 0 || rotary_dim > hd || rotary_dim <= 0))
    GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store_partials: rotary_dim %d for head_dim %d", rotary_dim, hd);
  if (page_size <= 0) GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store_partials: page_size %d", page_size);
  if (splits < 1 || hd <= 0 || hd > 2048) GB_FAIL(GB_ERR_ARG, "gb_qk_norm_rope_store_partials: %d splits, head_dim %d", splits, hd);
  const int slots = heads + (write_kv ? 2 * kv_heads : 0);
  const long long warps = (long long)n_tokens * slots;
  // The partial tiles go through shared memory in 16-byte pieces when rows and heads are aligned
  // for it and the copies fit; else every lane adds its columns with plain loads.
  const size_t smem_async = (size_t)4 * hd * (splits + 1) * sizeof(float);
  const int async_copies = (hd % 4 == 0 && ((uintptr_t)ws & 15) == 0 && smem_async <= 48 * 1024) ? 1 : 0;
  gb_launch(qk_norm_rope_store_partials_kernel, dim3(gb_div_up(warps, 4)), dim3(128),
            async_copies ? smem_async : (size_t)4 * hd * sizeof(float),
            stream, ws, splits, bias, (bf16*)q_out, q_gain, k_gain, eps, inv_freq, rotary_dim, adjacent, tok_req,
            tok_pos, block_table, bt_stride, page_size, (bf16*)k_pages, (bf16*)v_pages, n_pages, n_tokens, heads,
            kv_heads, hd, write_kv, async_copies, status);
  GB_CHECK_LAUNCH("gb_qk_norm_rope_store_partials");
  return GB_OK;
}

GB_API int gb_paged_attention(const void* q, int dtype, long long ldq, const void* k_pages, const void* v_pages,
                              const int* block_table, int bt_stride, int page_size, int n_pages, const int* tok_req,
                              const int* tok_pos, void* out, long long ldo, int n_tokens, int heads, int kv_heads,
                              int hd, float scale, float softcap, int window, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return GB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0)
    GB_FAIL(GB_ERR_ARG, "gb_paged_attention: %d heads over %d kv heads", heads, kv_heads);
  if (hd <= 0 || hd > 256) GB_FAIL(GB_ERR_ARG, "gb_paged_attention: head_dim %d outside 1..256", hd);
  if (page_size <= 0) GB_FAIL(GB_ERR_ARG, "gb_paged_attention: page_size %d", page_size);
  if (dtype == GB_F32)
    launch_attention<float>(q, ldq, k_pages, v_pages, block_table, bt_stride, page_size, n_pages, tok_req, tok_pos,
                            out, ldo, n_tokens, heads, kv_heads, hd, scale, softcap, window, status, stream);
  else if (dtype == GB_BF16)
    launch_attention<bf16>(q, ldq, k_pages, v_pages, block_table, bt_stride, page_size, n_pages, tok_req, tok_pos,
                           out, ldo, n_tokens, heads, kv_heads, hd, scale, softcap, window, status, stream);
  else
    GB_FAIL(GB_ERR_ARG, "gb_paged_attention: unknown dtype %d", dtype);
  GB_CHECK_LAUNCH("gb_paged_attention");
  return GB_OK;
}
