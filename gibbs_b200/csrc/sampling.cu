// Sampling of one token per logits row, on the device.
//
// Rules (MisterTK/gibbs src/runtime/lm.rs:1043-1235):
//  - temperature <= 1e-4: the index of the first maximum; NaN never wins.
//  - otherwise: the top k candidates (k <= 64) ordered by (logit descending,
//    id ascending); softmax of logit/temperature over them with the maximum
//    subtracted; the shortest prefix whose cumulative probability reaches
//    clamp(top_p, 0.01, 1); draw r = u * (sum of the kept probabilities) and
//    take the first candidate whose cumulative probability reaches r.
// The reference derives u from a hash of the recent tokens; here u comes from
// a counter-based generator (SplitMix64 of seed and draw counter) so that a
// seed reproduces a run.
#include "common.cuh"

namespace {

constexpr int MAX_K = 64;

struct Cand {
  float v;
  int id;
};

// a before b in (value descending, id ascending) order; id < 0 marks "none"
__device__ __forceinline__ bool better(const Cand& a, const Cand& b) {
  if (a.id < 0) return false;
  if (b.id < 0) return true;
  return a.v > b.v || (a.v == b.v && a.id < b.id);
}

__device__ __forceinline__ Cand warp_best(Cand c) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Cand other;
    other.v = __shfl_xor_sync(0xffffffffu, c.v, o);
    other.id = __shfl_xor_sync(0xffffffffu, c.id, o);
    if (better(other, c)) c = other;
  }
  return c;
}

// f(value, id) for every element of a row, each thread taking every blockDim-th group of four
// (or single element when the row cannot be read in 16-byte pieces).  Eight loads are requested
// before the first is used: a thread that waits for each load in turn spends the row's sixteen
// memory latencies one after the other.  The loads go through L2 (a row is read once).
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* x, int vocab, bool vec, F f) {
  const int T = blockDim.x;
  const int n4 = vec ? vocab >> 2 : 0;
  for (int i0 = threadIdx.x; i0 < n4; i0 += 8 * T) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i0 + u * T < n4) v[u] = __ldcg(reinterpret_cast<const float4*>(x) + i0 + u * T);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * T;
      if (i < n4) {
        f(v[u].x, 4 * i);
        f(v[u].y, 4 * i + 1);
        f(v[u].z, 4 * i + 2);
        f(v[u].w, 4 * i + 3);
      }
    }
  }
  for (int i0 = 4 * n4 + threadIdx.x; i0 < vocab; i0 += 8 * T) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i0 + u * T < vocab) v[u] = __ldcg(x + i0 + u * T);
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i0 + u * T < vocab) f(v[u], i0 + u * T);
  }
}

__device__ __forceinline__ float uniform24(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// ---- the top k of a row without k passes over it ----------------------------------------
// 1. every thread keeps the best of its own elements (one pass);
// 2. L = the k-th largest of these per-thread maxima (radix select in shared memory): k threads hold an
//    element >= L, so the k-th largest element of the row is >= L and all of the top k are >= L;
// 3. the elements >= L are collected (second pass; at most k - 1 threads hold elements above L, so they are
//    few unless values tie) and sorted by (logit descending, id ascending);
// 4. the first k are the candidates.  If more than SEL_CAP elements pass (thousands of equal values at the
//    threshold), the row falls back to k passes: never a wrong result.
constexpr int SEL_CAP = 4096;

// larger float <-> larger unsigned; 0 stands for "no element" (below -inf's key)
__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void sample_kernel(const float* logits, long long ldv, int vocab,
                              const float* temperature, const int* top_k,
                              const float* top_p, const unsigned long long* __restrict__ seed,
                              const long long* __restrict__ counter, int* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  __shared__ Cand warp_c[32];
  __shared__ Cand picked[MAX_K];
  __shared__ Cand prev;
  __shared__ Cand cand[SEL_CAP];
  __shared__ unsigned local_key[1024];
  __shared__ int hist[256];
  __shared__ unsigned sel_prefix;
  __shared__ int sel_need, n_cand;
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ldv;
  const float temp = temperature ? temperature[row] : 0.f;
  const bool greedy = !(temp > 1e-4f);
  int k = greedy ? 1 : (top_k ? top_k[row] : 50);
  k = k < 1 ? 1 : (k > MAX_K ? MAX_K : k);
  if (k > vocab) k = vocab;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int T = blockDim.x;
  const bool vec = (ldv % 4 == 0) && (((uintptr_t)logits & 15) == 0);

  // 1. this thread's best element
  Cand mine = {0.f, -1};
  for_each_logit(x, vocab, vec, [&](float v, int id) {
    const Cand c = {v, id};
    if (v == v && better(c, mine)) mine = c;                 // NaN never wins
  });
  local_key[threadIdx.x] = mine.id >= 0 ? ordered_key(mine.v) : 0u;
  if (threadIdx.x == 0) {
    sel_prefix = 0u;
    sel_need = k;
    n_cand = 0;
  }
  // 2. the k-th largest of the T keys, eight bits at a time from the top
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += T) hist[i] = 0;
    __syncthreads();
    const unsigned key = local_key[threadIdx.x], pre = sel_prefix;
    const unsigned above = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
    if ((key & above) == (pre & above)) atomicAdd(&hist[(key >> shift) & 255u], 1);
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins 255 - 8l down to 248 - 8l; find the bin in which the count from the top reaches `need`
      int mine8 = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) mine8 += hist[255 - 8 * lane - j];
      int incl = mine8;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const int need = sel_need, before = incl - mine8;
      if (before < need && need <= incl) {                 // exactly one lane
        int cum = before;
        for (int j = 0; j < 8; ++j) {
          const int bin = 255 - 8 * lane - j;
          if (cum + hist[bin] >= need) {
            sel_prefix = pre | ((unsigned)bin << shift);
            sel_need = need - cum;
            break;
          }
          cum += hist[bin];
        }
      }
    }
    __syncthreads();
  }
  const unsigned l_key = sel_prefix;                         // 0 when fewer than k threads hold an element
  // 3. everything >= L
  for_each_logit(x, vocab, vec, [&](float v, int id) {
    if (v == v && ordered_key(v) >= l_key) {
      const int at = atomicAdd(&n_cand, 1);
      if (at < SEL_CAP) cand[at] = Cand{v, id};
    }
  });
  __syncthreads();
  const int n = n_cand;
  int len = 0;
  if (n <= SEL_CAP) {
    // sort the candidates, best first (bitonic over the next power of two, padded with "none")
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    for (int i = n + threadIdx.x; i < n2; i += T) cand[i] = Cand{0.f, -1};
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int idx = threadIdx.x; idx < (n2 >> 1); idx += T) {
          const int i = 2 * idx - (idx & (stride - 1)), j = i + stride;
          const bool first_best = (i & size) == 0;
          const Cand a = cand[i], b2 = cand[j];
          if (better(b2, a) == first_best) {
            cand[i] = b2;
            cand[j] = a;
          }
        }
        __syncthreads();
      }
    }
    len = n < k ? n : k;
    if (threadIdx.x < len) picked[threadIdx.x] = cand[threadIdx.x];
    __syncthreads();
  } else {
    // k passes: each takes the best element that is worse than the one before
    for (int round = 0; round < k; ++round) {
      Cand best = {0.f, -1};
      const Cand p = prev;  // meaningful from the second pass on
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = x[i];
        if (v != v) continue;  // NaN never wins
        if (round > 0 && !(v < p.v || (v == p.v && i > p.id))) continue;
        const Cand c = {v, i};
        if (better(c, best)) best = c;
      }
      best = warp_best(best);
      if (lane == 0) warp_c[warp] = best;
      __syncthreads();
      if (warp == 0) {
        Cand c = lane < nwarps ? warp_c[lane] : Cand{0.f, -1};
        c = warp_best(c);
        if (lane == 0) {
          prev = c;
          if (c.id >= 0) picked[round] = c;
        }
      }
      __syncthreads();
      if (prev.id < 0) break;
      len = round + 1;
    }
  }

  if (threadIdx.x != 0) return;
  if (len == 0) {  // nothing above -inf that is not NaN
    out[row] = 0;
    return;
  }
  if (greedy) {
    out[row] = picked[0].id;
    return;
  }
  float probs[MAX_K];
  float mx = -INFINITY;
  for (int i = 0; i < len; ++i) mx = fmaxf(mx, picked[i].v / temp);
  float sum = 0.f;
  for (int i = 0; i < len; ++i) {
    probs[i] = expf(picked[i].v / temp - mx);
    sum += probs[i];
  }
  const float denom = fmaxf(sum, 1e-12f);
  for (int i = 0; i < len; ++i) probs[i] /= denom;
  float pt = top_p ? top_p[row] : 0.9f;
  pt = fminf(fmaxf(pt, 0.01f), 1.0f);
  int cut = len;
  float cum = 0.f;
  for (int i = 0; i < len; ++i) {
    cum += probs[i];
    if (cum >= pt) {
      cut = i + 1;
      break;
    }
  }
  float active = 0.f;
  for (int i = 0; i < cut; ++i) active += probs[i];
  const float r = uniform24(seed ? seed[row] : 0ull, counter ? (unsigned long long)counter[row] : 0ull) * active;
  cum = 0.f;
  int choice = picked[cut - 1].id;
  for (int i = 0; i < cut; ++i) {
    cum += probs[i];
    if (cum >= r) {
      choice = picked[i].id;
      break;
    }
  }
  out[row] = choice;
}

// All rows greedy: one pass, the first maximum of each row.
__global__ void argmax_kernel(const float* logits, long long ldv, int vocab, int* __restrict__ out) {
  __shared__ Cand warp_c[32];
  pdl_trigger();
  pdl_wait();
  const float* x = logits + (size_t)blockIdx.x * ldv;
  Cand best = {0.f, -1};
  const bool vec = (ldv % 4 == 0) && (((uintptr_t)logits & 15) == 0);
  for_each_logit(x, vocab, vec, [&](float v, int id) {
    const Cand c = {v, id};
    if (v == v && better(c, best)) best = c;
  });
  best = warp_best(best);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (lane == 0) warp_c[warp] = best;
  __syncthreads();
  if (warp == 0) {
    Cand c = lane < nwarps ? warp_c[lane] : Cand{0.f, -1};
    c = warp_best(c);
    if (lane == 0) out[blockIdx.x] = c.id < 0 ? 0 : c.id;
  }
}

// The same over a cluster of ARGMAX_CLUSTER blocks per row: each block scans its slice of the row
// and leaves its best in the first block's shared memory (a store through distributed shared
// memory); after the cluster barrier the first block picks among them.  (value, id) is a total
// order, so the result does not depend on which block found what.
constexpr int ARGMAX_CLUSTER = 8;

__global__ void __cluster_dims__(ARGMAX_CLUSTER, 1, 1) __launch_bounds__(512)
argmax_cluster_kernel(const float* logits, long long ldv, int vocab, int* __restrict__ out) {
  __shared__ Cand warp_c[32];
  __shared__ Cand block_c[ARGMAX_CLUSTER];
  pdl_trigger();
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int row = blockIdx.x / ARGMAX_CLUSTER;
  // slices of whole 16-byte pieces
  const int per = (((vocab + ARGMAX_CLUSTER - 1) / ARGMAX_CLUSTER) + 3) & ~3;
  const int lo = min(vocab, (int)rank * per), hi = min(vocab, lo + per);
  const float* x = logits + (size_t)row * ldv;
  const bool vec = (ldv % 4 == 0) && (((uintptr_t)logits & 15) == 0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  pdl_wait();
  Cand best = {0.f, -1};
  for_each_logit(x + lo, hi - lo, vec, [&](float v, int id) {
    const Cand c = {v, lo + id};
    if (v == v && better(c, best)) best = c;
  });
  best = warp_best(best);
  if (lane == 0) warp_c[warp] = best;
  __syncthreads();
  if (warp == 0) {
    Cand c = lane < nwarps ? warp_c[lane] : Cand{0.f, -1};
    c = warp_best(c);
    if (lane == 0) {
      const unsigned local = (unsigned)__cvta_generic_to_shared(&block_c[rank]);
      unsigned remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0u));
      asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(remote), "r"(__float_as_uint(c.v)), "r"(c.id)
                   : "memory");
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (rank == 0 && threadIdx.x == 0) {
    Cand c = block_c[0];
#pragma unroll
    for (int i = 1; i < ARGMAX_CLUSTER; ++i)
      if (better(block_c[i], c)) c = block_c[i];
    out[row] = c.id < 0 ? 0 : c.id;
  }
}

// Repetition penalty (MisterTK/gibbs src/runtime/lm.rs:1074-1108 for the greedy rule, :1163-1190
// for the sampling rule): a token that occurs c times among a row's recent tokens has its logit
// divided by the penalty when positive, multiplied when not, c times; the greedy rule then
// subtracts 1.5 * c, the sampling rule subtracts 1.5 after each of the c steps.  Applied in place
// to the logits row before the pick; rows whose penalty is <= 1 are left alone.
// recent: [rows][RECENT_MAX] token ids, -1 where a row has fewer.  One block per row, a thread
// per recent position; the first occurrence of a token does the work for all of them.
constexpr int RECENT_MAX = 64;

__global__ void repetition_penalty_kernel(float* logits, long long ldv, int vocab, const int* recent,
                                          const float* penalty, const float* temperature) {
  __shared__ int toks[RECENT_MAX];
  pdl_trigger();
  const int row = blockIdx.x, j = threadIdx.x;
  const int tok = recent[row * RECENT_MAX + j];
  const float pen = penalty[row];
  toks[j] = tok;
  __syncthreads();
  pdl_wait();
  if (!(pen > 1.0f) || tok < 0 || tok >= vocab) return;
  int count = 0;
  bool first = true;
  for (int i = 0; i < RECENT_MAX; ++i) {
    if (toks[i] == tok) {
      ++count;
      if (i < j) first = false;
    }
  }
  if (!first) return;
  const bool greedy = temperature == nullptr || temperature[row] <= 1e-4f;
  float* at = logits + (size_t)row * ldv + tok;
  float v = *at;
  for (int c = 0; c < count; ++c) {
    v = v > 0.f ? v / pen : v * pen;
    if (!greedy) v -= 1.5f;
  }
  if (greedy) v -= (float)count * 1.5f;
  *at = v;
}

// What a row's distribution says about a picked token (MisterTK/gibbs logprob_info,
// src/scheduler/mod.rs:272-315): the picked token's probability, the exact entropy of
// softmax(logits) (terms below 1e-12 dropped, as there) and the k most probable tokens, by (logit
// descending, id ascending).  One block per row; the candidates are found one after the other (k
// block-wide maxima): the report is asked for a handful of tokens, not for speed.
constexpr int MAX_LOGPROBS = 32;

__global__ void logprob_info_kernel(const float* logits, long long ldv, int vocab, const int* chosen, int k,
                                    float* __restrict__ chosen_prob, float* __restrict__ entropy,
                                    int* __restrict__ top_ids, float* __restrict__ top_probs) {
  __shared__ Cand warp_c[32];
  __shared__ float warp_f[32];
  __shared__ float bcast[2];
  __shared__ int taken[MAX_LOGPROBS];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ldv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  auto block_best = [&](Cand c) {
    c = warp_best(c);
    __syncthreads();
    if (lane == 0) warp_c[warp] = c;
    __syncthreads();
    Cand b = lane < nwarps ? warp_c[lane] : Cand{0.f, -1};
    return warp_best(b);                      // (every warp computes the same result)
  };
  auto block_sum_f = [&](float v) {
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) warp_f[warp] = v;
    __syncthreads();
    float t = lane < nwarps ? warp_f[lane] : 0.f;
    return warp_sum(t);
  };
  // the k best, one after the other
  for (int j = 0; j < k; ++j) {
    Cand best = {0.f, -1};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = x[i];
      bool free_ = v == v;
      for (int t = 0; t < j; ++t) free_ = free_ && taken[t] != i;
      const Cand c = {v, i};
      if (free_ && better(c, best)) best = c;
    }
    best = block_best(best);
    if (threadIdx.x == 0) {
      taken[j] = best.id;
      if (j == 0) bcast[0] = best.id >= 0 ? best.v : 0.f;     // the row's maximum
    }
    __syncthreads();
  }
  const float max_l = bcast[0];
  float se = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (v == v) se += expf(v - max_l);
  }
  se = block_sum_f(se);
  const float lse = max_l + logf(se);
  float ent = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (v == v) {
      const float p = expf(v - lse);
      if (p > 1e-12f) ent += p * (v - lse);
    }
  }
  ent = block_sum_f(ent);
  if (threadIdx.x == 0) {
    entropy[row] = -ent;
    const int c = chosen[row];
    const float lc = (c >= 0 && c < vocab) ? x[c] : max_l;
    chosen_prob[row] = fminf(expf(lc - lse), 1.0f);
  }
  if (threadIdx.x < k) {
    const int id = taken[threadIdx.x];
    top_ids[(size_t)row * k + threadIdx.x] = id;
    top_probs[(size_t)row * k + threadIdx.x] = id >= 0 ? expf(x[id] - lse) : 0.f;
  }
}

}  // namespace

// For each row: the probability of chosen[row] under softmax(logits[row]), the entropy of that
// distribution, and its k most probable tokens with their probabilities ([rows, k] each; -1 / 0 where
// a row has fewer than k numbers).  k in 1..32.
GB_API int gb_logprob_info(const float* logits, long long ldv, int rows, int vocab, const int* chosen, int k,
                           float* chosen_prob, float* entropy, int* top_ids, float* top_probs, cudaStream_t stream) {
  if (rows <= 0) return GB_OK;
  if (vocab <= 0) GB_FAIL(GB_ERR_ARG, "gb_logprob_info: vocabulary of %d", vocab);
  if (k < 1 || k > MAX_LOGPROBS) GB_FAIL(GB_ERR_ARG, "gb_logprob_info: %d candidates outside 1..%d", k, MAX_LOGPROBS);
  int threads = 64;
  while (threads < 1024 && threads * 8 < vocab) threads <<= 1;
  gb_launch(logprob_info_kernel, dim3(rows), dim3(threads), 0, stream, logits, ldv, vocab, chosen, k, chosen_prob,
            entropy, top_ids, top_probs);
  GB_CHECK_LAUNCH("gb_logprob_info");
  return GB_OK;
}

// logits: [rows, vocab] 32-bit with row stride ldv.  temperature / top_k /
// top_p / seed / counter are per row (null: greedy, 50, 0.9, 0, 0).
GB_API int gb_sample(const float* logits, long long ldv, int rows, int vocab, const float* temperature,
                     const int* top_k, const float* top_p, const unsigned long long* seed, const long long* counter,
                     int* out, cudaStream_t stream) {
  if (rows <= 0) return GB_OK;
  if (vocab <= 0) GB_FAIL(GB_ERR_ARG, "gb_sample: vocabulary of %d", vocab);
  int threads = 64;
  while (threads < 1024 && threads * 8 < vocab) threads <<= 1;
  if (temperature == nullptr) {
    if (vocab >= 8192 && rows * ARGMAX_CLUSTER <= 148) {
      // a large row and so few of them that a block per row would leave most SMs idle: eight blocks
      // share a row (6.4 against 12.7 us for 8 rows of 65,536; at 64 rows a block per row is faster)
      int th = 64;
      while (th < 512 && th * 8 * ARGMAX_CLUSTER < vocab) th <<= 1;
      gb_launch(argmax_cluster_kernel, dim3(rows * ARGMAX_CLUSTER), dim3(th), 0, stream, logits, ldv, vocab, out);
    } else {
      gb_launch(argmax_kernel, dim3(rows), dim3(threads), 0, stream, logits, ldv, vocab, out);
    }
    GB_CHECK_LAUNCH("gb_sample (argmax)");
    return GB_OK;
  }
  gb_launch(sample_kernel, dim3(rows), dim3(threads), 0, stream, logits, ldv, vocab, temperature, top_k, top_p, seed, counter, out);
  GB_CHECK_LAUNCH("gb_sample");
  return GB_OK;
}

// logits [rows, vocab] (row stride ldv) float32, changed in place; recent [rows, 64] int32 (-1:
// none); penalty [rows] float32; temperature [rows] float32 or null (all rows greedy).
GB_API int gb_repetition_penalty(float* logits, long long ldv, int vocab, const int* recent, const float* penalty,
                                 const float* temperature, int rows, cudaStream_t stream) {
  if (rows <= 0) return GB_OK;
  if (vocab <= 0) GB_FAIL(GB_ERR_ARG, "gb_repetition_penalty: vocabulary of %d", vocab);
  gb_launch(repetition_penalty_kernel, dim3(rows), dim3(RECENT_MAX), 0, stream, logits, ldv, vocab, recent, penalty,
            temperature);
  GB_CHECK_LAUNCH("gb_repetition_penalty");
  return GB_OK;
}
