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

__device__ __forceinline__ float uniform24(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void sample_kernel(const float* __restrict__ logits, long long ldv, int vocab,
                              const float* __restrict__ temperature, const int* __restrict__ top_k,
                              const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                              const long long* __restrict__ counter, int* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  __shared__ Cand warp_c[32];
  __shared__ Cand picked[MAX_K];
  __shared__ Cand prev;
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ldv;
  const float temp = temperature ? temperature[row] : 0.f;
  const bool greedy = !(temp > 1e-4f);
  int k = greedy ? 1 : (top_k ? top_k[row] : 50);
  k = k < 1 ? 1 : (k > MAX_K ? MAX_K : k);
  if (k > vocab) k = vocab;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

  int len = 0;
  for (int round = 0; round < k; ++round) {
    Cand best = {0.f, -1};
    const Cand p = prev;  // meaningful from round 1 on
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
__global__ void argmax_kernel(const float* __restrict__ logits, long long ldv, int vocab, int* __restrict__ out) {
  __shared__ Cand warp_c[32];
  pdl_trigger();
  pdl_wait();
  const float* x = logits + (size_t)blockIdx.x * ldv;
  Cand best = {0.f, -1};
  const bool vec = (ldv % 4 == 0) && (((uintptr_t)logits & 15) == 0);
  const int n4 = vec ? vocab >> 2 : 0;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const Cand c = {e[k], 4 * i + k};
      if (e[k] == e[k] && better(c, best)) best = c;
    }
  }
  for (int i = 4 * n4 + threadIdx.x; i < vocab; i += blockDim.x) {
    const Cand c = {x[i], i};
    if (c.v == c.v && better(c, best)) best = c;
  }
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

}  // namespace

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
    gb_launch(argmax_kernel, dim3(rows), dim3(threads), 0, stream, logits, ldv, vocab, out);
    GB_CHECK_LAUNCH("gb_sample (argmax)");
    return GB_OK;
  }
  gb_launch(sample_kernel, dim3(rows), dim3(threads), 0, stream, logits, ldv, vocab, temperature, top_k, top_p, seed, counter, out);
  GB_CHECK_LAUNCH("gb_sample");
  return GB_OK;
}
