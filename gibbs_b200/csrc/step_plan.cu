// The host side of a step as data: a list of operations (embed, norm, matrix product, short
// convolution, q/k norm + rotation + cache write, attention, SwiGLU) with their buffers and
// constants, built once per model, and one function that walks the list and launches the kernels
// of a step.  A step then costs one call from Python instead of some hundred and fifty, each of
// which spent more time in the interpreter than its kernel runs on the GPU.
//
// What changes from step to step are a few numbers and addresses ("symbols": tokens, requests,
// wanted rows, the longest portion and context, whether every request brings one token, where the
// step's metadata and its logits lie).  An operand of an operation is either a constant or names a
// symbol.  Decisions that depend on the step's sizes are taken here exactly as the Python wrappers
// take them (gibbs_b200/ops): whether a product splits K and leaves partial tiles for the kernel
// after it, which attention kernel runs and into how many CTAs the keys are split.
//
// The kernels live in the other libraries; their entry points are handed over once as a table of
// function pointers (gb_plan_bind), so this file launches nothing by itself and knows no model.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace {

// ---- entry points of the kernel libraries (signatures as in their sources) ----
typedef int (*EmbedFn)(const void*, int, const int*, float*, int, int, int, cudaStream_t);
typedef int (*RmsnormFn)(float*, long long, const float*, void*, int, const int*, int, int, float, const float*, int,
                         long long, const float*, cudaStream_t);
typedef int (*LinearSimtFn)(const void*, int, long long, const void*, int, long long, const float*, void*, int,
                            long long, int, int, int, int, cudaStream_t);
typedef int (*LinearTcFn)(const void*, long long, const void*, long long, const float*, void*, int, long long, int, int,
                          int, float*, int, int, int*, cudaStream_t);
typedef int (*LinearTcSplitsFn)(int, int, int);
typedef int (*ShortConvFn)(const void*, int, long long, const float*, const float*, float*, long long, const int*,
                           const int*, const int*, const int*, void*, int, int, int, int, int, cudaStream_t);
typedef int (*ShortConvPartialsFn)(const float*, int, long long, const float*, const float*, const float*, float*,
                                   long long, const int*, const int*, void*, int, int, int, cudaStream_t);
typedef int (*QkRopeFn)(void*, int, long long, const float*, const float*, float, const float*, int, int, const int*,
                        const int*, const int*, int, int, void*, void*, int, int, int, int, int, int, int*, cudaStream_t);
typedef int (*QkRopePartialsFn)(const float*, int, const float*, void*, const float*, const float*, float, const float*,
                                int, int, const int*, const int*, const int*, int, int, void*, void*, int, int, int, int,
                                int, int, int*, cudaStream_t);
typedef int (*PagedAttentionFn)(const void*, int, long long, const void*, const void*, const int*, int, int, int,
                                const int*, const int*, void*, long long, int, int, int, int, float, int, int*,
                                cudaStream_t);
typedef int (*AttentionTcFn)(const void*, long long, const void*, const void*, const int*, int, int, int, const int*,
                             const int*, const int*, void*, long long, int, int, int, int, int, int, float, int, int,
                             float*, int*, cudaStream_t);
typedef int (*AttentionTcgen05Fn)(const void*, long long, const void*, const void*, const int*, int, int, int,
                                  const int*, const int*, const int*, void*, long long, int, int, int, int, int, float,
                                  int, int*, cudaStream_t);
typedef int (*AttentionTcgen05SupportedFn)(int, int, int, int, long long, long long);
typedef int (*SwigluFn)(const void*, void*, int, int, int, cudaStream_t);

enum Fn : int { F_EMBED = 0, F_RMSNORM, F_LINEAR_SIMT, F_LINEAR_TC, F_LINEAR_TC_SPLITS, F_SHORT_CONV,
                F_SHORT_CONV_PARTIALS, F_QKROPE, F_QKROPE_PARTIALS, F_PAGED_ATTENTION, F_ATTENTION_TC,
                F_ATTENTION_TCGEN05, F_ATTENTION_TCGEN05_SUPPORTED, F_SWIGLU, F_COUNT };
// which library an entry point belongs to (0: core, 1: tensor cores), for the caller to fetch the message
const int FN_LIB[F_COUNT] = {0, 0, 0, 1, 1, 0, 0, 0, 0, 0, 1, 1, 1, 0};
void* g_fn[F_COUNT];

enum Op : int { P_EMBED = 1, P_RMSNORM = 2, P_LINEAR = 3, P_SHORT_CONV = 4, P_QKROPE = 5, P_ATTENTION = 6, P_SWIGLU = 7 };
enum Sym : int { S_N = 0, S_R, S_W, S_MAXQ, S_MAXCTX, S_ONE_EACH, S_TOKEN_IDS, S_TOK_REQ, S_TOK_POS, S_Q_START, S_Q_LEN,
                 S_START_POS, S_CTX_LEN, S_SLOT_IDS, S_WANT_ROWS, S_LOGITS, S_BLOCK_TABLE0, S_COUNT = 32 };
constexpr long long SYM_BIT = 1ll << 62;

enum LinearFlag : int { LF_RESIDUAL = 1, LF_PARTIALS_IF_ONE_EACH = 2, LF_PARTIALS = 4 };

struct PlanOp {              // 224 bytes; the meaning of a[] per operation is given where it is executed
  int op;
  int flags;
  long long a[24];
  double f[3];
};
static_assert(sizeof(PlanOp) == 224, "operation size");

struct Walk {
  const long long* sym;
  cudaStream_t stream;
  int* status;
  float* ws;                 // shared workspace of split-K partial tiles
  float* attn_ws;            // workspace of the decode attention's key splits
  int attn_ctas;             // how many CTAs the decode attention aims for
  int tc_flags;              // flags of the tensor-core product (evict-first hint)
  int use_tcgen05;
  int defer_whole_rows;      // from this many rows on, an unsplit product into the residual is deferred whole
  // what the operation before left for the one after it
  int pend_splits; const float* pend_bias;     // partial sums to be added to the residual by the next norm
  int part_splits; const float* part_bias;     // partial tiles of a product whose consumer adds them itself
  const void* q; long long ldq;                // where the rotated queries lie
  int launches;
  int failed_lib;
};

inline long long val(const Walk& w, long long v) { return (v & SYM_BIT) ? w.sym[v & 0xffff] : v; }
template <typename T> inline T* ptr(const Walk& w, long long v) { return reinterpret_cast<T*>(val(w, v)); }

#define PLAN_CALL(w, fn_index, expr)                 \
  do {                                               \
    const int rc_ = (expr);                          \
    if (rc_ < 0) {                                   \
      (w).failed_lib = FN_LIB[fn_index];             \
      return rc_;                                    \
    }                                                \
    (w).launches += rc_ > 0 ? rc_ : 1;               \
  } while (0)

int attention_splits(const Walk& w, int n_requests, int kv_heads, int max_ctx_len) {
  int by_sm = w.attn_ctas / (n_requests * kv_heads > 0 ? n_requests * kv_heads : 1);
  if (by_sm < 1) by_sm = 1;
  int by_len = (max_ctx_len + 127) / 128;
  if (by_len < 1) by_len = 1;
  // up to 16 splits of at least two tiles; beyond that (up to the merge kernel's 32) only with 1,024 keys a split
  int s = by_len < 16 ? by_len : 16;
  int by_long = max_ctx_len / 1024;
  if (by_long > 32) by_long = 32;
  if (by_long > s) s = by_long;
  if (s > by_sm) s = by_sm;
  return s < 1 ? 1 : s;
}

int run_op(Walk& w, const PlanOp& o) {
  const long long* a = o.a;
  const int N = (int)w.sym[S_N], R = (int)w.sym[S_R], W = (int)w.sym[S_W];
  const int one_each = (int)w.sym[S_ONE_EACH];
  switch (o.op) {
    case P_EMBED: {
      // a0 table, a1 its dtype, a2 out (f32 [., dim]), a3 dim, a4 vocabulary
      PLAN_CALL(w, F_EMBED, ((EmbedFn)g_fn[F_EMBED])(ptr<const void>(w, a[0]), (int)a[1], ptr<const int>(w, SYM_BIT | S_TOKEN_IDS),
                                                      ptr<float>(w, a[2]), N, (int)a[3], (int)a[4], w.stream));
      return 0;
    }
    case P_RMSNORM: {
      // a0 x (f32), a1 its row stride, a2 gain, a3 out, a4 out dtype, a5 gather the wanted rows (0/1), a6 dim; f0 eps
      const bool gather = a[5] != 0;
      const int n_rows = gather ? W : N;
      if (n_rows <= 0) return 0;                               // (a step that wants no logits)
      const float* pend = w.pend_splits > 0 ? w.ws : nullptr;
      PLAN_CALL(w, F_RMSNORM, ((RmsnormFn)g_fn[F_RMSNORM])(
          ptr<float>(w, a[0]), a[1], ptr<const float>(w, a[2]), ptr<void>(w, a[3]), (int)a[4],
          gather ? ptr<const int>(w, SYM_BIT | S_WANT_ROWS) : nullptr, n_rows, (int)a[6], (float)o.f[0], pend,
          w.pend_splits, (long long)N, pend ? w.pend_bias : nullptr, w.stream));
      w.pend_splits = 0;
      return 0;
    }
    case P_LINEAR: {
      // a0 x, a1 its row stride, a2 W, a3 its row stride, a4 bias, a5 out, a6 its row stride, a7 rows (N or W, a
      // symbol), a8 n, a9 k, a10 kernel (0 tensor cores, 1 FFMA), a11 mode (0 bf16, 1 f32, 2 add into f32, 3 SwiGLU),
      // a12 x dtype, a13 W dtype, a14 out dtype
      const int M = (int)val(w, a[7]);
      if (M <= 0) return 0;
      const float* bias = ptr<const float>(w, a[4]);
      if (a[10] == 0) {
        const int n = (int)a[8], k = (int)a[9];
        const int splits = ((LinearTcSplitsFn)g_fn[F_LINEAR_TC_SPLITS])(M, n, k);
        const bool wants = (o.flags & LF_RESIDUAL) || (o.flags & LF_PARTIALS) ||
                           ((o.flags & LF_PARTIALS_IF_ONE_EACH) && one_each);
        // a large unsplit product into the residual stream is deferred as a whole (ops.DEFER_WHOLE_ROWS)
        const bool whole = (o.flags & LF_RESIDUAL) && splits == 1 && M >= w.defer_whole_rows;
        const bool defer = (wants && splits > 1 && (a[11] == 0 || a[11] == 2)) || whole;
        PLAN_CALL(w, F_LINEAR_TC, ((LinearTcFn)g_fn[F_LINEAR_TC])(
            ptr<const void>(w, a[0]), a[1], ptr<const void>(w, a[2]), a[3], bias, ptr<void>(w, a[5]), (int)a[11], a[6],
            M, n, k, (splits > 1 || whole) ? w.ws : nullptr, whole ? 2 : (defer ? 1 : 0), w.tc_flags, w.status,
            w.stream));
        if (o.flags & LF_RESIDUAL) {
          w.pend_splits = defer ? splits : 0;
          w.pend_bias = bias;
        } else {
          w.part_splits = defer ? splits : 0;
          w.part_bias = bias;
        }
      } else {
        PLAN_CALL(w, F_LINEAR_SIMT, ((LinearSimtFn)g_fn[F_LINEAR_SIMT])(
            ptr<const void>(w, a[0]), (int)a[12], a[1], ptr<const void>(w, a[2]), (int)a[13], a[3], bias,
            ptr<void>(w, a[5]), (int)a[14], a[6], a[11] == 2 ? 1 : 0, M, (int)a[8], (int)a[9], w.stream));
        if (o.flags & LF_RESIDUAL) w.pend_splits = 0; else w.part_splits = 0;
      }
      return 0;
    }
    case P_SHORT_CONV: {
      // a0 [B | C | x] rows, a1 their stride, a2 taps, a3 conv bias, a4 state of slot 0, a5 elements between slots,
      // a6 out, a7 hidden, a8 taps per channel, a9 dtype
      if (w.part_splits > 0 && one_each) {
        PLAN_CALL(w, F_SHORT_CONV_PARTIALS, ((ShortConvPartialsFn)g_fn[F_SHORT_CONV_PARTIALS])(
            w.ws, w.part_splits, (long long)N, w.part_bias, ptr<const float>(w, a[2]), ptr<const float>(w, a[3]),
            ptr<float>(w, a[4]), a[5], ptr<const int>(w, SYM_BIT | S_SLOT_IDS), ptr<const int>(w, SYM_BIT | S_Q_START),
            ptr<void>(w, a[6]), R, (int)a[7], (int)a[8], w.stream));
      } else {
        PLAN_CALL(w, F_SHORT_CONV, ((ShortConvFn)g_fn[F_SHORT_CONV])(
            ptr<const void>(w, a[0]), (int)a[9], a[1], ptr<const float>(w, a[2]), ptr<const float>(w, a[3]),
            ptr<float>(w, a[4]), a[5], ptr<const int>(w, SYM_BIT | S_SLOT_IDS), ptr<const int>(w, SYM_BIT | S_TOK_REQ),
            ptr<const int>(w, SYM_BIT | S_Q_START), ptr<const int>(w, SYM_BIT | S_Q_LEN), ptr<void>(w, a[6]), N, R,
            (int)a[7], (int)a[8], (int)w.sym[S_MAXQ], w.stream));
      }
      w.part_splits = 0;
      return 0;
    }
    case P_QKROPE: {
      // a0 [q | k | v] rows, a1 their stride, a2 q gain, a3 k gain, a4 inv_freq, a5 rotary_dim, a6 adjacent pairs,
      // a7 block-table group, a8 page size, a9 k pages, a10 v pages, a11 pages, a12 heads, a13 kv heads, a14 head_dim,
      // a15 writes k/v, a16 dtype, a17 q of the partial-tile variant, a18 entries per request in a block table; f0 eps
      const int* bt = ptr<const int>(w, SYM_BIT | (S_BLOCK_TABLE0 + a[7]));
      if (w.part_splits > 0) {
        PLAN_CALL(w, F_QKROPE_PARTIALS, ((QkRopePartialsFn)g_fn[F_QKROPE_PARTIALS])(
            w.ws, w.part_splits, w.part_bias, ptr<void>(w, a[17]), ptr<const float>(w, a[2]), ptr<const float>(w, a[3]),
            (float)o.f[0], ptr<const float>(w, a[4]), (int)a[5], (int)a[6], ptr<const int>(w, SYM_BIT | S_TOK_REQ),
            ptr<const int>(w, SYM_BIT | S_TOK_POS), bt, (int)a[18], (int)a[8], ptr<void>(w, a[9]), ptr<void>(w, a[10]),
            (int)a[11], N, (int)a[12], (int)a[13], (int)a[14], (int)a[15], w.status, w.stream));
        w.q = ptr<const void>(w, a[17]);
        w.ldq = a[12] * a[14];
      } else {
        PLAN_CALL(w, F_QKROPE, ((QkRopeFn)g_fn[F_QKROPE])(
            ptr<void>(w, a[0]), (int)a[16], a[1], ptr<const float>(w, a[2]), ptr<const float>(w, a[3]), (float)o.f[0],
            ptr<const float>(w, a[4]), (int)a[5], (int)a[6], ptr<const int>(w, SYM_BIT | S_TOK_REQ),
            ptr<const int>(w, SYM_BIT | S_TOK_POS), bt, (int)a[18], (int)a[8], ptr<void>(w, a[9]), ptr<void>(w, a[10]),
            (int)a[11], N, (int)a[12], (int)a[13], (int)a[14], (int)a[15], w.status, w.stream));
        w.q = ptr<const void>(w, a[0]);
        w.ldq = a[1];
      }
      w.part_splits = 0;
      return 0;
    }
    case P_ATTENTION: {
      // a0 out, a1 its row stride, a2 k pages, a3 v pages, a4 block-table group, a5 page size, a6 pages, a7 heads,
      // a8 kv heads, a9 head_dim, a10 window, a11 dtype, a12 entries per request in a block table; f0 scale
      const int heads = (int)a[7], kvh = (int)a[8], hd = (int)a[9], page_size = (int)a[5];
      const int group = heads / kvh;
      const int* bt = ptr<const int>(w, SYM_BIT | (S_BLOCK_TABLE0 + a[4]));
      const float scale = (float)o.f[0];
      void* out = ptr<void>(w, a[0]);
      const bool tc = a[11] == GB_BF16 && g_fn[F_ATTENTION_TC] != nullptr && hd % 16 == 0 && hd >= 16 && hd <= 128 &&
                      heads % kvh == 0 && group <= 64 && w.ldq % 8 == 0 && a[1] % 2 == 0 && ((uintptr_t)w.q & 15) == 0;
      if (!tc) {
        PLAN_CALL(w, F_PAGED_ATTENTION, ((PagedAttentionFn)g_fn[F_PAGED_ATTENTION])(
            w.q, (int)a[11], w.ldq, ptr<const void>(w, a[2]), ptr<const void>(w, a[3]), bt, (int)a[12], page_size,
            (int)a[6], ptr<const int>(w, SYM_BIT | S_TOK_REQ), ptr<const int>(w, SYM_BIT | S_TOK_POS), out, a[1], N,
            heads, kvh, hd, scale, (int)a[10], w.status, w.stream));
        return 0;
      }
      const int max_q = (int)w.sym[S_MAXQ];
      const bool small = (long long)max_q * group <= 16 && group <= 16;
      if (!small && w.use_tcgen05 && scale > 0.f && ((uintptr_t)out & 15) == 0 &&
          ((AttentionTcgen05SupportedFn)g_fn[F_ATTENTION_TCGEN05_SUPPORTED])(heads, kvh, hd, page_size, w.ldq, a[1])) {
        PLAN_CALL(w, F_ATTENTION_TCGEN05, ((AttentionTcgen05Fn)g_fn[F_ATTENTION_TCGEN05])(
            w.q, w.ldq, ptr<const void>(w, a[2]), ptr<const void>(w, a[3]), bt, (int)a[12], page_size, (int)a[6],
            ptr<const int>(w, SYM_BIT | S_Q_START), ptr<const int>(w, SYM_BIT | S_Q_LEN),
            ptr<const int>(w, SYM_BIT | S_START_POS), out, a[1], R, N, heads, kvh, hd, scale, (int)a[10], w.status,
            w.stream));
        return 0;
      }
      const int splits = small ? attention_splits(w, R, kvh, (int)w.sym[S_MAXCTX]) : 1;
      PLAN_CALL(w, F_ATTENTION_TC, ((AttentionTcFn)g_fn[F_ATTENTION_TC])(
          w.q, w.ldq, ptr<const void>(w, a[2]), ptr<const void>(w, a[3]), bt, (int)a[12], page_size, (int)a[6],
          ptr<const int>(w, SYM_BIT | S_Q_START), ptr<const int>(w, SYM_BIT | S_Q_LEN),
          ptr<const int>(w, SYM_BIT | S_START_POS), out, a[1], R, N, max_q, heads, kvh, hd, scale, (int)a[10], splits,
          splits > 1 ? w.attn_ws : nullptr, w.status, w.stream));
      return 0;
    }
    case P_SWIGLU: {
      // a0 [g | u] rows, a1 out, a2 dtype, a3 inner
      PLAN_CALL(w, F_SWIGLU, ((SwigluFn)g_fn[F_SWIGLU])(ptr<const void>(w, a[0]), ptr<void>(w, a[1]), (int)a[2], N, (int)a[3],
                                                         w.stream));
      return 0;
    }
  }
  snprintf(gb_error_buffer(), 512, "gb_plan_run: unknown operation %d", o.op);
  w.failed_lib = 2;
  return GB_ERR_ARG;
}

}  // namespace

// The table of entry points, in the order of the enumeration above (null where a library is not loaded).
GB_API int gb_plan_bind(void* const* fns, int n) {
  if (n != F_COUNT) GB_FAIL(GB_ERR_ARG, "gb_plan_bind: %d entry points, %d expected", n, (int)F_COUNT);
  memcpy(g_fn, fns, sizeof(g_fn));
  return GB_OK;
}

GB_API int gb_plan_op_bytes() { return (int)sizeof(PlanOp); }

struct GbPlanRun {
  const void* ops; int n_ops;
  const long long* sym; int n_sym;
  float* ws; float* attn_ws; int* status;
  int attn_ctas, tc_flags, use_tcgen05, defer_whole_rows;
  int failed_lib;            // out: 0 core, 1 tensor cores, 2 this library (where the message of a failure lies)
};

// Launches the kernels of one step.  Returns the number of kernels launched, or a negative error code.
GB_API int gb_plan_run(GbPlanRun* r, cudaStream_t stream) {
  if (r->n_sym < S_COUNT) GB_FAIL(GB_ERR_ARG, "gb_plan_run: %d symbols, %d expected", r->n_sym, (int)S_COUNT);
  Walk w;
  memset(&w, 0, sizeof(w));
  w.sym = r->sym; w.stream = stream; w.status = r->status; w.ws = r->ws; w.attn_ws = r->attn_ws;
  w.attn_ctas = r->attn_ctas; w.tc_flags = r->tc_flags; w.use_tcgen05 = r->use_tcgen05;
  w.defer_whole_rows = r->defer_whole_rows;
  w.failed_lib = 2;
  const PlanOp* ops = (const PlanOp*)r->ops;
  for (int i = 0; i < r->n_ops; ++i) {
    const int rc = run_op(w, ops[i]);
    if (rc < 0) {
      r->failed_lib = w.failed_lib;
      return rc;
    }
  }
  return w.launches;
}
