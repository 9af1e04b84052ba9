// Gated short convolution over a ragged batch: for every request its next
// n tokens (a prompt portion or one decoded token) continue a depthwise
// causal convolution whose last K-1 inputs live in the request's state slot.
//
//   bx[t, c]  = B[t, c] * x[t, c]                       (rows of [B | C | x])
//   cv[t, c]  = sum_j taps[c, j] * win[(K-1) + i - (K-1-j), c] (+ bias[c])
//               win = [state (K-1 rows); bx of this request (n rows)], i = t's
//               index among the request's tokens: tap K-1 multiplies the
//               current token, tap 0 the oldest
//   out[t, c] = C[t, c] * cv[t, c]
//   state    <- last K-1 rows of win
// (MisterTK/gibbs arch/lib/transformer.json5:140-151; src/graph/cpu.rs:952-994.)
//
// Two launches: outputs first (token-parallel, read the old state), then the
// state update (one thread per request and channel).  The state holds the
// 32-bit products B*x, so decoding from it repeats the prompt pass exactly.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void short_conv_out_kernel(const T* bcx, long long ld, const float* __restrict__ taps,
                                      const float* __restrict__ bias, const float* state,
                                      long long slot_stride, const int* slot_ids,
                                      const int* tok_req, const int* q_start,
                                      T* __restrict__ out, int n_tokens, int hidden, int K) {
  pdl_trigger();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_tokens * hidden) return;
  const int t = (int)(gid / hidden), c = (int)(gid - (long long)t * hidden);
  const int r = tok_req[t];
  const int first = q_start[r];
  const int i = t - first;
  const float* st = state + (size_t)slot_ids[r] * slot_stride;
  float acc = 0.f;
  for (int j = 0; j < K; ++j) {
    const int src = i - (K - 1 - j);
    float v;
    if (src >= 0) {
      const T* row = bcx + (size_t)(first + src) * ld;
      v = to_f32(row[c]) * to_f32(row[2 * hidden + c]);
    } else {
      v = st[(size_t)(K - 1 + src) * hidden + c];
    }
    acc = fmaf(taps[(size_t)c * K + j], v, acc);
  }
  if (bias) acc += bias[c];
  out[(size_t)t * hidden + c] = from_f32<T>(to_f32(bcx[(size_t)t * ld + hidden + c]) * acc);
}

// The same for bfloat16 rows whose width is a multiple of 8: one thread takes 8 neighbouring
// channels of a token with 16-byte loads and stores.
__global__ void short_conv_out_vec8_kernel(const bf16* bcx, long long ld, const float* __restrict__ taps,
                                           const float* __restrict__ bias, const float* state,
                                           long long slot_stride, const int* slot_ids,
                                           const int* tok_req, const int* q_start,
                                           bf16* __restrict__ out, int n_tokens, int hidden, int K) {
  pdl_trigger();
  pdl_wait();
  const int groups = hidden >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_tokens * groups) return;
  const int t = (int)(gid / groups), c = (int)(gid - (long long)t * groups) << 3;
  const int r = tok_req[t];
  const int first = q_start[r];
  const int i = t - first;
  const float* st = state + (size_t)slot_ids[r] * slot_stride;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  auto unpack = [](uint4 u, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(h[e]);
      f[2 * e] = v.x;
      f[2 * e + 1] = v.y;
    }
  };
  for (int j = 0; j < K; ++j) {
    const int src = i - (K - 1 - j);
    float v[8];
    if (src >= 0) {
      const bf16* row = bcx + (size_t)(first + src) * ld;
      float b[8], x[8];
      unpack(*reinterpret_cast<const uint4*>(row + c), b);
      unpack(*reinterpret_cast<const uint4*>(row + 2 * hidden + c), x);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = b[e] * x[e];
    } else {
      const float4* sp = reinterpret_cast<const float4*>(st + (size_t)(K - 1 + src) * hidden + c);
      const float4 s0 = sp[0], s1 = sp[1];
      v[0] = s0.x; v[1] = s0.y; v[2] = s0.z; v[3] = s0.w; v[4] = s1.x; v[5] = s1.y; v[6] = s1.z; v[7] = s1.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = fmaf(taps[(size_t)(c + e) * K + j], v[e], acc[e]);
  }
  float g[8];
  unpack(*reinterpret_cast<const uint4*>(bcx + (size_t)t * ld + hidden + c), g);
  uint4 o;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float a0 = acc[2 * e] + (bias ? bias[c + 2 * e] : 0.f), a1 = acc[2 * e + 1] + (bias ? bias[c + 2 * e + 1] : 0.f);
    oh[e] = __floats2bfloat162_rn(g[2 * e] * a0, g[2 * e + 1] * a1);
  }
  *reinterpret_cast<uint4*>(out + (size_t)t * hidden + c) = o;
}

// The same for narrow filters (K <= 4), eight consecutive tokens per thread: the products B*x a
// filter position needs are kept in registers while the window slides along the tokens, so every
// row of [B | C | x] is read once instead of K times and the taps once per thread.  Where the run
// crosses into another request the window restarts from that request's state.  The terms are
// added in the order of the kernels above (oldest tap first), so the results are the same bits.
template <int K>
__global__ void short_conv_out_run_kernel(const bf16* bcx, long long ld, const float* __restrict__ taps,
                                          const float* __restrict__ bias, const float* state,
                                          long long slot_stride, const int* slot_ids,
                                          const int* tok_req, const int* q_start,
                                          bf16* __restrict__ out, int n_tokens, int hidden) {
  constexpr int RUN = 8;
  pdl_trigger();
  const int groups = hidden >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long n_runs = ((long long)n_tokens + RUN - 1) / RUN;
  if (gid >= n_runs * groups) return;
  const int run = (int)(gid / groups), c = (int)(gid - (long long)run * groups) << 3;
  auto unpack = [](uint4 u, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(h[e]);
      f[2 * e] = v.x;
      f[2 * e + 1] = v.y;
    }
  };
  float tap[K][8], bs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
#pragma unroll
    for (int j = 0; j < K; ++j) tap[j][e] = taps[(size_t)(c + e) * K + j];
    bs[e] = bias ? bias[c + e] : 0.f;
  }
  float win[K][8];                                           // win[j]: the product that meets tap j for the current token
  const int t0 = run * RUN, t1 = min(t0 + RUN, n_tokens);
  // Taps, bias and the step's metadata (which request a token belongs to, where the request starts
  // in the batch, its state slot) do not come from the product in front: they are read before the
  // wait for it.  Behind the wait all rows of the run, and the K-1 older positions of its first
  // token, are requested before the first is used (a thread that fetched them one by one would spend
  // as many memory latencies one after the other).
  int rreq[RUN];
#pragma unroll
  for (int u = 0; u < RUN; ++u) rreq[u] = tok_req[t0 + u < t1 ? t0 + u : t1 - 1];
  int cur_req = rreq[0], first = q_start[cur_req];
  const float* st0 = state + (size_t)slot_ids[cur_req] * slot_stride;
  gb_pin(first);
  gb_pin(st0);
#pragma unroll
  for (int u = 0; u < RUN; ++u) gb_pin(rreq[u]);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
#pragma unroll
    for (int j = 0; j < K; ++j) gb_pin(tap[j][e]);
    gb_pin(bs[e]);
  }
  pdl_wait();
  uint4 rb[RUN], rx[RUN], rg[RUN];
#pragma unroll
  for (int u = 0; u < RUN; ++u) {
    const int t = t0 + u < t1 ? t0 + u : t1 - 1;
    const bf16* row = bcx + (size_t)t * ld;
    rb[u] = __ldcg(reinterpret_cast<const uint4*>(row + c));
    rx[u] = __ldcg(reinterpret_cast<const uint4*>(row + 2 * hidden + c));
    rg[u] = __ldcg(reinterpret_cast<const uint4*>(row + hidden + c));
  }
  {
    // the K-1 older positions of the run's first token: earlier tokens of its request in the batch, or its state
    const int i0 = t0 - first;
    uint4 ob[K - 1], ox[K - 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      const int src = i0 - (K - 1 - j);
      if (src >= 0) {
        const bf16* prow = bcx + (size_t)(first + src) * ld;
        ob[j] = __ldcg(reinterpret_cast<const uint4*>(prow + c));
        ox[j] = __ldcg(reinterpret_cast<const uint4*>(prow + 2 * hidden + c));
      } else {
        const uint4* sp = reinterpret_cast<const uint4*>(st0 + (size_t)(K - 1 + src) * hidden + c);
        ob[j] = __ldcg(sp);
        ox[j] = __ldcg(sp + 1);
      }
    }
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      if (i0 - (K - 1 - j) >= 0) {
        float pb[8], px[8];
        unpack(ob[j], pb);
        unpack(ox[j], px);
#pragma unroll
        for (int e = 0; e < 8; ++e) win[j][e] = pb[e] * px[e];
      } else {
        win[j][0] = __uint_as_float(ob[j].x); win[j][1] = __uint_as_float(ob[j].y);
        win[j][2] = __uint_as_float(ob[j].z); win[j][3] = __uint_as_float(ob[j].w);
        win[j][4] = __uint_as_float(ox[j].x); win[j][5] = __uint_as_float(ox[j].y);
        win[j][6] = __uint_as_float(ox[j].z); win[j][7] = __uint_as_float(ox[j].w);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < RUN; ++u) {
    const int t = t0 + u;
    if (t >= t1) break;
    const int r = rreq[u];
    const bool restart = r != cur_req;                       // (never the run's first token: it is prepared above)
    if (restart) {
      cur_req = r;
      first = q_start[r];
    }
    const int i = t - first;
    float b[8], x[8], g[8];
    unpack(rb[u], b);
    unpack(rx[u], x);
    unpack(rg[u], g);
    if (restart) {
      // the K-1 older positions: earlier tokens of this request in the batch, or its state
      const float* st = state + (size_t)slot_ids[r] * slot_stride;
#pragma unroll
      for (int j = 0; j < K - 1; ++j) {
        const int src = i - (K - 1 - j);
        if (src >= 0) {
          const bf16* prow = bcx + (size_t)(first + src) * ld;
          float pb[8], px[8];
          unpack(*reinterpret_cast<const uint4*>(prow + c), pb);
          unpack(*reinterpret_cast<const uint4*>(prow + 2 * hidden + c), px);
#pragma unroll
          for (int e = 0; e < 8; ++e) win[j][e] = pb[e] * px[e];
        } else {
          const float4* sp = reinterpret_cast<const float4*>(st + (size_t)(K - 1 + src) * hidden + c);
          const float4 s0 = sp[0], s1 = sp[1];
          win[j][0] = s0.x; win[j][1] = s0.y; win[j][2] = s0.z; win[j][3] = s0.w;
          win[j][4] = s1.x; win[j][5] = s1.y; win[j][6] = s1.z; win[j][7] = s1.w;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) win[K - 1][e] = b[e] * x[e];
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) a = fmaf(tap[j][e], win[j][e], a);
      acc[e] = a + bs[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(g[2 * e] * acc[2 * e], g[2 * e + 1] * acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)t * hidden + c) = o;
    // slide: the next token's tap j meets what tap j+1 met now
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) win[j][e] = win[j + 1][e];
  }
}

template <typename T>
__global__ void short_conv_state_kernel(const T* bcx, long long ld, float* __restrict__ state,
                                        long long slot_stride, const int* slot_ids,
                                        const int* q_start, const int* q_len,
                                        int n_requests, int hidden, int K) {
  pdl_trigger();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_requests * hidden) return;
  const int r = (int)(gid / hidden), c = (int)(gid - (long long)r * hidden);
  const int n = q_len[r], first = q_start[r];
  if (n <= 0) return;
  float* st = state + (size_t)slot_ids[r] * slot_stride;
  // new[j] = win[n + j]: an old state row while n + j < K-1 (read above the
  // row being written, so ascending j is safe in place), else a new product.
  for (int j = 0; j < K - 1; ++j) {
    const int w = n + j;
    float v;
    if (w < K - 1) {
      v = st[(size_t)w * hidden + c];
    } else {
      const T* row = bcx + (size_t)(first + w - (K - 1)) * ld;
      v = to_f32(row[c]) * to_f32(row[2 * hidden + c]);
    }
    st[(size_t)j * hidden + c] = v;
  }
}

// Every request brings exactly one token: output and state update in one pass,
// one thread per request and channel (it alone reads and writes its state column).
// KT: the kernel width when it is 2, 3 or 4 (the loops unroll and the window stays in registers), else 0.
template <typename T, int KT>
__global__ void short_conv_decode_kernel(const T* bcx, long long ld, const float* __restrict__ taps,
                                         const float* __restrict__ bias, float* __restrict__ state,
                                         long long slot_stride, const int* slot_ids,
                                         const int* q_start, T* __restrict__ out, int n_requests,
                                         int hidden, int K_) {
  const int K = KT ? KT : K_;
  pdl_trigger();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_requests * hidden) return;
  const int r = (int)(gid / hidden), c = (int)(gid - (long long)r * hidden);
  // Metadata, taps and the state an earlier step left are read before the wait for the kernel in
  // front; after it only this step's [B | C | x] row is missing.
  int t = q_start[r];
  gb_pin(t);
  float* st = state + (size_t)slot_ids[r] * slot_stride;
  float old[KT ? KT : MAX_TAPS], tap[KT ? KT : MAX_TAPS];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) old[j] = st[(size_t)j * hidden + c];
#pragma unroll
  for (int j = 0; j < K; ++j) tap[j] = taps[(size_t)c * K + j];
  float cb = bias ? bias[c] : 0.f;
  const T* row = bcx + (size_t)t * ld;
#pragma unroll
  for (int j = 0; j < K - 1; ++j) gb_pin(old[j]);
#pragma unroll
  for (int j = 0; j < K; ++j) gb_pin(tap[j]);
  gb_pin(cb);
  gb_pin(row);
  gb_pin(st);
  pdl_wait();
  // (ldcg_now and not __ldcg, which for bfloat16 is an asm the compiler may move above the wait)
  const float bx = to_f32(ldcg_now(row + c)) * to_f32(ldcg_now(row + 2 * hidden + c));
  const float gate = to_f32(ldcg_now(row + hidden + c));
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    acc = fmaf(tap[j], old[j], acc);
    if (j > 0) st[(size_t)(j - 1) * hidden + c] = old[j];      // shift the window by one
  }
  acc = fmaf(tap[K - 1], bx, acc);
  st[(size_t)(K - 2) * hidden + c] = bx;
  if (bias) acc += cb;
  out[(size_t)t * hidden + c] = from_f32<T>(gate * acc);
}

// The same, reading [B | C | x] as the partial tiles of the split-K product that made it
// (ws[split][token][3*hidden], 32-bit, plus in_bias): their sum is rounded to bfloat16 exactly
// where the product's own reduction would have rounded it, then used as above.
template <int KT>
__global__ void short_conv_decode_partials_kernel(const float* ws, int splits, long long n_rows,
                                                  const float* __restrict__ in_bias, const float* __restrict__ taps,
                                                  const float* __restrict__ bias, float* __restrict__ state,
                                                  long long slot_stride, const int* slot_ids,
                                                  const int* q_start, bf16* __restrict__ out,
                                                  int n_requests, int hidden, int K_) {
  const int K = KT ? KT : K_;
  pdl_trigger();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n_requests * hidden) return;
  const int r = (int)(gid / hidden), c = (int)(gid - (long long)r * hidden);
  // Metadata, taps, biases and the state an earlier step left are read before the wait for the
  // product in front; after it only its partial tiles are missing (one trip to L2).
  int t = q_start[r];
  gb_pin(t);
  const size_t ld = (size_t)3 * hidden;
  const size_t at[3] = {(size_t)t * ld + c, (size_t)t * ld + hidden + c, (size_t)t * ld + 2 * hidden + c};
  float* st = state + (size_t)slot_ids[r] * slot_stride;
  float old[KT ? KT : MAX_TAPS], tap[KT ? KT : MAX_TAPS];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) old[j] = st[(size_t)j * hidden + c];
#pragma unroll
  for (int j = 0; j < K; ++j) tap[j] = taps[(size_t)c * K + j];
  float cb = bias ? bias[c] : 0.f;
  float ib[3] = {0.f, 0.f, 0.f};
  if (in_bias) {
    ib[0] = in_bias[c];
    ib[1] = in_bias[hidden + c];
    ib[2] = in_bias[2 * hidden + c];
  }
#pragma unroll
  for (int j = 0; j < K - 1; ++j) gb_pin(old[j]);
#pragma unroll
  for (int j = 0; j < K; ++j) gb_pin(tap[j]);
  gb_pin(cb);
  gb_pin(ib[0]); gb_pin(ib[1]); gb_pin(ib[2]);
  gb_pin(st);
  bf16* o = out + (size_t)t * hidden + c;
  gb_pin(o);                                                 // (addresses too are ready before the wait)
  pdl_wait();
  float v[3];
  sum_partials<3>(ws, splits, (size_t)n_rows * ld, at, v);
  if (in_bias) {
    v[0] += ib[0];
    v[1] += ib[1];
    v[2] += ib[2];
  }
  const float bv = to_f32(from_f32<bf16>(v[0])), cv = to_f32(from_f32<bf16>(v[1])), xv = to_f32(from_f32<bf16>(v[2]));
  const float bx = bv * xv;
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    acc = fmaf(tap[j], old[j], acc);
    if (j > 0) st[(size_t)(j - 1) * hidden + c] = old[j];
  }
  acc = fmaf(tap[K - 1], bx, acc);
  st[(size_t)(K - 2) * hidden + c] = bx;
  if (bias) acc += cb;
  *o = __float2bfloat16_rn(cv * acc);
}

}  // namespace

// One token per request, with [B | C | x] given as the `splits` partial tiles of a split-K product
// (ws: 32-bit [splits][n_rows][3*hidden], in_bias: its bias or null); out is bfloat16.
GB_API int gb_short_conv_partials(const float* ws, int splits, long long n_rows, const float* in_bias,
                                  const float* taps, const float* bias, float* state, long long slot_stride,
                                  const int* slot_ids, const int* q_start, void* out, int n_requests, int hidden, int K,
                                  cudaStream_t stream) {
  if (n_requests <= 0) return 0;
  if (K < 2 || K > MAX_TAPS) GB_FAIL(GB_ERR_ARG, "gb_short_conv_partials: kernel width %d outside 2..%d", K, MAX_TAPS);
  if (splits < 1) GB_FAIL(GB_ERR_ARG, "gb_short_conv_partials: %d splits", splits);
  const long long total = (long long)n_requests * hidden;
  auto kernel = K == 2 ? short_conv_decode_partials_kernel<2>
                : K == 3 ? short_conv_decode_partials_kernel<3>
                : K == 4 ? short_conv_decode_partials_kernel<4> : short_conv_decode_partials_kernel<0>;
  gb_launch(kernel, dim3(gb_div_up(total, 128)), dim3(128), 0, stream, ws, splits, n_rows,
            in_bias, taps, bias, state, slot_stride, slot_ids, q_start, (bf16*)out, n_requests, hidden, K);
  GB_CHECK_LAUNCH("gb_short_conv_partials");
  return 1;
}

// bcx: [n_tokens, 3*hidden] rows of [B | C | x] with row stride ld; taps
// [hidden, K] and bias [hidden] (optional) in 32-bit; state: 32-bit, slot s at
// state + s*slot_stride holding [K-1, hidden]; out: [n_tokens, hidden].  max_q_len: the longest
// portion of the batch if the host knows it (0: unknown).  Returns the number of kernels launched.
GB_API int gb_short_conv(const void* bcx, int dtype, long long ld, const float* taps, const float* bias,
                         float* state, long long slot_stride, const int* slot_ids, const int* tok_req,
                         const int* q_start, const int* q_len, void* out, int n_tokens, int n_requests, int hidden,
                         int K, int max_q_len, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (K < 2 || K > MAX_TAPS) GB_FAIL(GB_ERR_ARG, "gb_short_conv: kernel width %d outside 2..%d", K, MAX_TAPS);
  const int threads = 256;
  if (max_q_len == 1 && n_tokens == n_requests) {           // one token per request
    const long long total = (long long)n_requests * hidden;
    if (dtype == GB_F32) {
      auto kernel = K == 2 ? short_conv_decode_kernel<float, 2> : K == 3 ? short_conv_decode_kernel<float, 3>
                    : K == 4 ? short_conv_decode_kernel<float, 4> : short_conv_decode_kernel<float, 0>;
      gb_launch(kernel, dim3(gb_div_up(total, threads)), dim3(threads), 0, stream, (const float*)bcx, ld, taps, bias,
                state, slot_stride, slot_ids, q_start, (float*)out, n_requests, hidden, K);
    } else if (dtype == GB_BF16) {
      auto kernel = K == 2 ? short_conv_decode_kernel<bf16, 2> : K == 3 ? short_conv_decode_kernel<bf16, 3>
                    : K == 4 ? short_conv_decode_kernel<bf16, 4> : short_conv_decode_kernel<bf16, 0>;
      gb_launch(kernel, dim3(gb_div_up(total, threads)), dim3(threads), 0, stream, (const bf16*)bcx, ld, taps, bias,
                state, slot_stride, slot_ids, q_start, (bf16*)out, n_requests, hidden, K);
    } else
      GB_FAIL(GB_ERR_ARG, "gb_short_conv: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("gb_short_conv (decode)");
    return 1;
  }
  const long long total = (long long)n_tokens * hidden;
  const long long total_s = (long long)n_requests * hidden;
  if (dtype == GB_F32) {
    gb_launch(short_conv_out_kernel<float>, dim3(gb_div_up(total, threads)), dim3(threads), 0, stream, (const float*)bcx, ld, taps, bias, state, slot_stride, slot_ids, tok_req, q_start, (float*)out, n_tokens,
        hidden, K);
    gb_launch(short_conv_state_kernel<float>, dim3(gb_div_up(total_s, threads)), dim3(threads), 0, stream, (const float*)bcx, ld, state, slot_stride, slot_ids, q_start, q_len, n_requests, hidden, K);
  } else if (dtype == GB_BF16) {
    const bool vec = hidden % 8 == 0 && ld % 8 == 0 && slot_stride % 4 == 0 && ((uintptr_t)bcx & 15) == 0 &&
                     ((uintptr_t)out & 15) == 0 && ((uintptr_t)state & 15) == 0;
    if (vec && K <= 4) {
      const long long work = (((long long)n_tokens + 7) / 8) * (hidden / 8);
      const dim3 grid(gb_div_up(work, 128)), block(128);
      if (K == 2)
        gb_launch(short_conv_out_run_kernel<2>, grid, block, 0, stream, (const bf16*)bcx, ld, taps, bias,
                  (const float*)state, slot_stride, slot_ids, tok_req, q_start, (bf16*)out, n_tokens, hidden);
      else if (K == 3)
        gb_launch(short_conv_out_run_kernel<3>, grid, block, 0, stream, (const bf16*)bcx, ld, taps, bias,
                  (const float*)state, slot_stride, slot_ids, tok_req, q_start, (bf16*)out, n_tokens, hidden);
      else
        gb_launch(short_conv_out_run_kernel<4>, grid, block, 0, stream, (const bf16*)bcx, ld, taps, bias,
                  (const float*)state, slot_stride, slot_ids, tok_req, q_start, (bf16*)out, n_tokens, hidden);
    } else if (vec)
      gb_launch(short_conv_out_vec8_kernel, dim3(gb_div_up(total / 8, threads)), dim3(threads), 0, stream,
                (const bf16*)bcx, ld, taps, bias, (const float*)state, slot_stride, slot_ids, tok_req, q_start,
                (bf16*)out, n_tokens, hidden, K);
    else
      gb_launch(short_conv_out_kernel<bf16>, dim3(gb_div_up(total, threads)), dim3(threads), 0, stream, (const bf16*)bcx, ld, taps, bias, state, slot_stride, slot_ids, tok_req, q_start, (bf16*)out, n_tokens,
        hidden, K);
    gb_launch(short_conv_state_kernel<bf16>, dim3(gb_div_up(total_s, threads)), dim3(threads), 0, stream, (const bf16*)bcx, ld, state, slot_stride, slot_ids, q_start, q_len, n_requests, hidden, K);
  } else {
    GB_FAIL(GB_ERR_ARG, "gb_short_conv: unknown dtype %d", dtype);
  }
  GB_CHECK_LAUNCH("gb_short_conv");
  return 2;
}
