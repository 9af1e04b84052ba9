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
//
// Operations beyond the built-in ones are registered by name at run time (gb_plan_register_op): a
// part that brings kernels of its own hands over one C function per operation, gets an id back,
// and emits records with that id; the walker calls the function with the record's operands
// (symbols already replaced by the step's values) and the stream.  Nothing here is edited for it.
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "common.cuh"
#include "gb_plan_op.h"

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
                                const int*, const int*, void*, long long, int, int, int, int, float, float, int, int*,
                                cudaStream_t);
typedef int (*ScaleSoftcapFn)(float*, long long, float, float, cudaStream_t);
typedef int (*AttentionTcFn)(const void*, long long, const void*, const void*, const int*, int, int, int, const int*,
                             const int*, const int*, void*, long long, int, int, int, int, int, int, float, int, int,
                             float*, int*, cudaStream_t);
typedef int (*AttentionTcgen05Fn)(const void*, long long, const void*, const void*, const int*, int, int, int,
                                  const int*, const int*, const int*, void*, long long, int, int, int, int, int, float,
                                  int, int*, cudaStream_t);
typedef int (*AttentionTcgen05SupportedFn)(int, int, int, int, long long, long long);
typedef int (*SwigluFn)(const void*, void*, int, int, int, cudaStream_t);
typedef int (*LinearDecodeFn)(const void*, long long, int, const float*, float, const int*, const float*, int,
                              long long, const void*, long long, const float*, void*, int, long long, int, int, int,
                              float*, long long, int, int*, cudaStream_t);
typedef int (*LinearDecodePartsFn)(int, int);
typedef int (*LinearDecodeSupportedFn)(int, const void*, long long, int);
typedef int (*LinearDecodeNormedOkFn)(int, int, int);
typedef int (*AddPendingFn)(float*, long long, const float*, int, const float*, long long, int, cudaStream_t);

enum Fn : int { F_EMBED = 0, F_RMSNORM, F_LINEAR_SIMT, F_LINEAR_TC, F_LINEAR_TC_SPLITS, F_SHORT_CONV,
                F_SHORT_CONV_PARTIALS, F_QKROPE, F_QKROPE_PARTIALS, F_PAGED_ATTENTION, F_ATTENTION_TC,
                F_ATTENTION_TCGEN05, F_ATTENTION_TCGEN05_SUPPORTED, F_SWIGLU, F_LINEAR_DECODE, F_LINEAR_DECODE_PARTS,
                F_LINEAR_DECODE_SUPPORTED, F_ADD_PENDING, F_LINEAR_DECODE_NORMED_OK, F_SCALE_SOFTCAP, F_COUNT };
// which library an entry point belongs to (0: core, 1: tensor cores), for the caller to fetch the message
const int FN_LIB[F_COUNT] = {0, 0, 0, 1, 1, 0, 0, 0, 0, 0, 1, 1, 1, 0, 1, 1, 1, 0, 1, 0};
void* g_fn[F_COUNT];

enum Op : int { P_EMBED = 1, P_RMSNORM = 2, P_LINEAR = 3, P_SHORT_CONV = 4, P_QKROPE = 5, P_ATTENTION = 6, P_SWIGLU = 7,
                P_SCALE_SOFTCAP = 8 };
// the step's symbols (gb_plan_op.h gives their meaning), under the short names used below
enum Sym : int { S_N = GB_SYM_TOKENS, S_R = GB_SYM_REQUESTS, S_W = GB_SYM_WANTED, S_MAXQ = GB_SYM_MAX_PORTION,
                 S_MAXCTX = GB_SYM_MAX_CONTEXT, S_ONE_EACH = GB_SYM_ONE_EACH, S_TOKEN_IDS = GB_SYM_TOKEN_IDS,
                 S_TOK_REQ = GB_SYM_TOKEN_REQUEST, S_TOK_POS = GB_SYM_TOKEN_POSITION, S_Q_START = GB_SYM_PORTION_START,
                 S_Q_LEN = GB_SYM_PORTION_LENGTH, S_START_POS = GB_SYM_LENGTH_BEFORE, S_CTX_LEN = GB_SYM_LENGTH_AFTER,
                 S_SLOT_IDS = GB_SYM_SLOT_IDS, S_WANT_ROWS = GB_SYM_WANTED_ROWS, S_LOGITS = GB_SYM_LOGITS,
                 S_BLOCK_TABLE0 = GB_SYM_BLOCK_TABLE0, S_TABLE_STRIDE = GB_SYM_TABLE_STRIDE, S_COUNT = GB_SYM_COUNT };
constexpr long long SYM_BIT = 1ll << 62;

enum LinearFlag : int { LF_RESIDUAL = 1, LF_PARTIALS_IF_ONE_EACH = 2, LF_PARTIALS = 4, LF_NORMED = 8 };
enum NormFlag : int { NF_LAZY = 1 };      // the product after it may run the norm itself (up to 64 rows)
constexpr int FIRST_REGISTERED_OP = 64;
constexpr int MAX_REGISTERED_OPS = 64;

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
  // products of decode size (csrc/gemm_tc_decode.cu)
  float* residual; long long residual_ld;      // the stream itself (for operations that need it whole)
  int decode_products;                         // products of up to this many rows run on the decode kernel (0: none)
  float* ssq;                                  // partial sums of squares of the stream's rows [parts][N]
  int ssq_parts;                               // > 0: ssq describes the stream as it stands
  const struct PlanOp* lazy_norm;              // a norm that was not launched: the next product runs it
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

int run_registered(Walk& w, const PlanOp& o);

int run_op(Walk& w, const PlanOp& o, bool force = false) {
  const long long* a = o.a;
  const int N = (int)w.sym[S_N], R = (int)w.sym[S_R], W = (int)w.sym[S_W];
  const int one_each = (int)w.sym[S_ONE_EACH];
  switch (o.op) {
    case P_EMBED: {
      // a0 table, a1 its dtype, a2 out (f32 [., dim]), a3 dim, a4 vocabulary
      w.ssq_parts = 0;
      PLAN_CALL(w, F_EMBED, ((EmbedFn)g_fn[F_EMBED])(ptr<const void>(w, a[0]), (int)a[1], ptr<const int>(w, SYM_BIT | S_TOKEN_IDS),
                                                      ptr<float>(w, a[2]), N, (int)a[3], (int)a[4], w.stream));
      return 0;
    }
    case P_RMSNORM: {
      // a0 x (f32), a1 its row stride, a2 gain, a3 out, a4 out dtype, a5 gather the wanted rows (0/1), a6 dim,
      // a7, a8 (with NF_LAZY) n and k of the product that reads the rows; f0 eps
      const bool gather = a[5] != 0;
      const int n_rows = gather ? W : N;
      if (n_rows <= 0) return 0;                               // (a step that wants no logits)
      if ((o.flags & NF_LAZY) && !force && n_rows <= w.decode_products && w.pend_splits == 0 && a[4] == GB_BF16 &&
          ((LinearDecodeNormedOkFn)g_fn[F_LINEAR_DECODE_NORMED_OK])(n_rows, (int)a[7], (int)a[8])) {
        w.lazy_norm = &o;                                      // the product that reads these rows normalises them
        return 0;
      }
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
      const PlanOp* lazy = (o.flags & LF_NORMED) ? w.lazy_norm : nullptr;
      w.lazy_norm = nullptr;
      if (a[10] == 0 && M <= w.decode_products &&
          ((LinearDecodeSupportedFn)g_fn[F_LINEAR_DECODE_SUPPORTED])(M, ptr<const void>(w, a[2]), a[3], (int)a[9])) {
        // up to 64 rows: K is split inside a cluster, and a norm that was left out runs inside the product
        const int n = (int)a[8], k = (int)a[9];
        const bool residual = (o.flags & LF_RESIDUAL) != 0;
        const void* x = ptr<const void>(w, a[0]);
        long long ldx = a[1];
        const float* gain = nullptr;
        const int* rows = nullptr;
        float eps = 0.f;
        if (lazy) {
          x = ptr<const void>(w, lazy->a[0]);
          ldx = lazy->a[1];
          gain = ptr<const float>(w, lazy->a[2]);
          eps = (float)lazy->f[0];
          rows = lazy->a[5] != 0 ? ptr<const int>(w, SYM_BIT | S_WANT_ROWS) : nullptr;
        }
        const int parts = residual ? ((LinearDecodePartsFn)g_fn[F_LINEAR_DECODE_PARTS])(n, k) : 0;
        PLAN_CALL(w, F_LINEAR_DECODE, ((LinearDecodeFn)g_fn[F_LINEAR_DECODE])(
            x, ldx, lazy ? 1 : 0, gain, eps, rows, (lazy && w.ssq_parts > 0) ? w.ssq : nullptr, w.ssq_parts,
            (long long)N, ptr<const void>(w, a[2]), a[3], bias, ptr<void>(w, a[5]), (int)a[11], a[6], M, n, k,
            residual ? w.ssq : nullptr, (long long)N, w.tc_flags, w.status, w.stream));
        if (residual) {
          w.pend_splits = 0;
          w.ssq_parts = parts;
        } else {
          w.part_splits = 0;
        }
        return 0;
      }
      if (lazy) {
        // the product cannot take the norm in: run it after all
        const int rc = run_op(w, *lazy, true);
        if (rc < 0) return rc;
      }
      if (o.flags & LF_RESIDUAL) w.ssq_parts = 0;
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
            ptr<const int>(w, SYM_BIT | S_TOK_POS), bt, (int)val(w, a[18]), (int)a[8], ptr<void>(w, a[9]), ptr<void>(w, a[10]),
            (int)a[11], N, (int)a[12], (int)a[13], (int)a[14], (int)a[15], w.status, w.stream));
        w.q = ptr<const void>(w, a[17]);
        w.ldq = a[12] * a[14];
      } else {
        PLAN_CALL(w, F_QKROPE, ((QkRopeFn)g_fn[F_QKROPE])(
            ptr<void>(w, a[0]), (int)a[16], a[1], ptr<const float>(w, a[2]), ptr<const float>(w, a[3]), (float)o.f[0],
            ptr<const float>(w, a[4]), (int)a[5], (int)a[6], ptr<const int>(w, SYM_BIT | S_TOK_REQ),
            ptr<const int>(w, SYM_BIT | S_TOK_POS), bt, (int)val(w, a[18]), (int)a[8], ptr<void>(w, a[9]), ptr<void>(w, a[10]),
            (int)a[11], N, (int)a[12], (int)a[13], (int)a[14], (int)a[15], w.status, w.stream));
        w.q = ptr<const void>(w, a[0]);
        w.ldq = a[1];
      }
      w.part_splits = 0;
      return 0;
    }
    case P_ATTENTION: {
      // a0 out, a1 its row stride, a2 k pages, a3 v pages, a4 block-table group, a5 page size, a6 pages, a7 heads,
      // a8 kv heads, a9 head_dim, a10 window, a11 dtype, a12 entries per request in a block table; f0 scale,
      // f1 soft cap of the scores (0: none; only the generic kernel applies one)
      const int heads = (int)a[7], kvh = (int)a[8], hd = (int)a[9], page_size = (int)a[5];
      const int group = heads / kvh;
      const int* bt = ptr<const int>(w, SYM_BIT | (S_BLOCK_TABLE0 + a[4]));
      const float scale = (float)o.f[0], softcap = (float)o.f[1];
      void* out = ptr<void>(w, a[0]);
      const bool tc = softcap <= 0.f && a[11] == GB_BF16 && g_fn[F_ATTENTION_TC] != nullptr && hd % 16 == 0 && hd >= 16 && hd <= 128 &&
                      heads % kvh == 0 && group <= 64 && w.ldq % 8 == 0 && a[1] % 2 == 0 && ((uintptr_t)w.q & 15) == 0;
      if (!tc) {
        PLAN_CALL(w, F_PAGED_ATTENTION, ((PagedAttentionFn)g_fn[F_PAGED_ATTENTION])(
            w.q, (int)a[11], w.ldq, ptr<const void>(w, a[2]), ptr<const void>(w, a[3]), bt, (int)val(w, a[12]), page_size,
            (int)a[6], ptr<const int>(w, SYM_BIT | S_TOK_REQ), ptr<const int>(w, SYM_BIT | S_TOK_POS), out, a[1], N,
            heads, kvh, hd, scale, softcap, (int)a[10], w.status, w.stream));
        return 0;
      }
      const int max_q = (int)w.sym[S_MAXQ];
      const bool small = (long long)max_q * group <= 16 && group <= 16;
      if (!small && w.use_tcgen05 && scale > 0.f && ((uintptr_t)out & 15) == 0 &&
          ((AttentionTcgen05SupportedFn)g_fn[F_ATTENTION_TCGEN05_SUPPORTED])(heads, kvh, hd, page_size, w.ldq, a[1])) {
        PLAN_CALL(w, F_ATTENTION_TCGEN05, ((AttentionTcgen05Fn)g_fn[F_ATTENTION_TCGEN05])(
            w.q, w.ldq, ptr<const void>(w, a[2]), ptr<const void>(w, a[3]), bt, (int)val(w, a[12]), page_size, (int)a[6],
            ptr<const int>(w, SYM_BIT | S_Q_START), ptr<const int>(w, SYM_BIT | S_Q_LEN),
            ptr<const int>(w, SYM_BIT | S_START_POS), out, a[1], R, N, heads, kvh, hd, scale, (int)a[10], w.status,
            w.stream));
        return 0;
      }
      const int splits = small ? attention_splits(w, R, kvh, (int)w.sym[S_MAXCTX]) : 1;
      PLAN_CALL(w, F_ATTENTION_TC, ((AttentionTcFn)g_fn[F_ATTENTION_TC])(
          w.q, w.ldq, ptr<const void>(w, a[2]), ptr<const void>(w, a[3]), bt, (int)val(w, a[12]), page_size, (int)a[6],
          ptr<const int>(w, SYM_BIT | S_Q_START), ptr<const int>(w, SYM_BIT | S_Q_LEN),
          ptr<const int>(w, SYM_BIT | S_START_POS), out, a[1], R, N, max_q, heads, kvh, hd, scale, (int)a[10], splits,
          splits > 1 ? w.attn_ws : nullptr, w.status, w.stream));
      return 0;
    }
    case P_SCALE_SOFTCAP: {
      // a0 the values (f32; the step's logits when it names that symbol), a1 columns, a2 rows (a symbol); f0 scale, f1 cap
      const long long rows = val(w, a[2]);
      if (rows <= 0) return 0;
      PLAN_CALL(w, F_SCALE_SOFTCAP, ((ScaleSoftcapFn)g_fn[F_SCALE_SOFTCAP])(ptr<float>(w, a[0]), rows * a[1], (float)o.f[0],
                                                                            (float)o.f[1], w.stream));
      return 0;
    }
    case P_SWIGLU: {
      // a0 [g | u] rows, a1 out, a2 dtype, a3 inner
      PLAN_CALL(w, F_SWIGLU, ((SwigluFn)g_fn[F_SWIGLU])(ptr<const void>(w, a[0]), ptr<void>(w, a[1]), (int)a[2], N, (int)a[3],
                                                         w.stream));
      return 0;
    }
  }
  if (o.op >= FIRST_REGISTERED_OP) return run_registered(w, o);
  snprintf(gb_error_buffer(), 512, "gb_plan_run: unknown operation %d", o.op);
  w.failed_lib = 2;
  return GB_ERR_ARG;
}

// ---- operations registered from outside ----
struct Registered {
  char name[64];
  GbPlanOpFn fn;
};
Registered g_registered[MAX_REGISTERED_OPS];
int g_n_registered = 0;

int run_registered(Walk& w, const PlanOp& o) {
  const int i = o.op - FIRST_REGISTERED_OP;
  if (i < 0 || i >= g_n_registered) {
    snprintf(gb_error_buffer(), 512, "gb_plan_run: operation %d is not registered", o.op);
    w.failed_lib = 2;
    return GB_ERR_ARG;
  }
  // such an operation sees the stream whole: what a product left to be added is added first, and
  // what this file remembers about the stream no longer holds afterwards
  if (w.pend_splits > 0) {
    const int N = (int)w.sym[S_N];
    PLAN_CALL(w, F_ADD_PENDING, ((AddPendingFn)g_fn[F_ADD_PENDING])(
        w.residual, w.residual_ld, w.ws, w.pend_splits, w.pend_bias, (long long)N, (int)w.residual_ld, w.stream));
    w.pend_splits = 0;
  }
  w.ssq_parts = 0;
  w.lazy_norm = nullptr;
  w.part_splits = 0;
  long long a[24];
  for (int j = 0; j < 24; ++j) a[j] = val(w, o.a[j]);
  GbPlanCtx ctx;
  ctx.stream = w.stream;
  ctx.status = w.status;
  ctx.sym = w.sym;
  ctx.n_sym = S_COUNT;
  const int rc = g_registered[i].fn(&ctx, a, o.f, o.flags);
  if (rc < 0) {
    snprintf(gb_error_buffer(), 512, "gb_plan_run: the registered operation '%s' failed with code %d",
             g_registered[i].name, rc);
    w.failed_lib = 2;
    return rc;
  }
  w.launches += rc;
  return 0;
}

}  // namespace

// Register an operation under a name; returns its id (the same id when the name is registered
// again, with the new function), or a negative error code.  The function gets the record's
// operands with symbols replaced by the step's values and returns the number of kernels it
// launched (on ctx->stream), or a negative code.
GB_API int gb_plan_register_op(const char* name, GbPlanOpFn fn) {
  if (name == nullptr || fn == nullptr || strlen(name) == 0 || strlen(name) >= sizeof(g_registered[0].name))
    GB_FAIL(GB_ERR_ARG, "gb_plan_register_op: a name of 1 to 63 characters and a function are needed");
  for (int i = 0; i < g_n_registered; ++i)
    if (strcmp(g_registered[i].name, name) == 0) {
      g_registered[i].fn = fn;
      return FIRST_REGISTERED_OP + i;
    }
  if (g_n_registered == MAX_REGISTERED_OPS)
    GB_FAIL(GB_ERR_ARG, "gb_plan_register_op: all %d places are taken", MAX_REGISTERED_OPS);
  strcpy(g_registered[g_n_registered].name, name);
  g_registered[g_n_registered].fn = fn;
  return FIRST_REGISTERED_OP + g_n_registered++;
}

// The id of a registered operation, or -1.
GB_API int gb_plan_op_id(const char* name) {
  for (int i = 0; i < g_n_registered; ++i)
    if (strcmp(g_registered[i].name, name) == 0) return FIRST_REGISTERED_OP + i;
  return -1;
}

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
  float* ssq; int decode_products;
  float* residual; long long residual_ld;
  // timing != 0: every operation is bracketed by CUDA events (which also keeps operations from
  // overlapping) and its time is added to label_ms[a[23]] of its record; for measurements only
  int timing; int n_labels;
  float* label_ms; int* label_count;
};

// Launches the kernels of one step.  Returns the number of kernels launched, or a negative error code.
GB_API int gb_plan_run(GbPlanRun* r, cudaStream_t stream) {
  if (r->n_sym < S_COUNT) GB_FAIL(GB_ERR_ARG, "gb_plan_run: %d symbols, %d expected", r->n_sym, (int)S_COUNT);
  Walk w;
  memset(&w, 0, sizeof(w));
  w.sym = r->sym; w.stream = stream; w.status = r->status; w.ws = r->ws; w.attn_ws = r->attn_ws;
  w.attn_ctas = r->attn_ctas; w.tc_flags = r->tc_flags; w.use_tcgen05 = r->use_tcgen05;
  w.defer_whole_rows = r->defer_whole_rows;
  w.ssq = r->ssq; w.decode_products = g_fn[F_LINEAR_DECODE] != nullptr ? r->decode_products : 0;
  w.residual = r->residual; w.residual_ld = r->residual_ld;
  w.failed_lib = 2;
  const PlanOp* ops = (const PlanOp*)r->ops;
  static std::vector<cudaEvent_t> events;      // timing mode: two per operation, made once
  if (r->timing) {
    while ((int)events.size() < 2 * r->n_ops) {
      cudaEvent_t e;
      GB_CUDA(cudaEventCreate(&e));
      events.push_back(e);
    }
  }
  for (int i = 0; i < r->n_ops; ++i) {
    if (r->timing) GB_CUDA(cudaEventRecord(events[2 * i], stream));
    const int rc = run_op(w, ops[i]);
    if (rc < 0) {
      r->failed_lib = w.failed_lib;
      return rc;
    }
    if (r->timing) GB_CUDA(cudaEventRecord(events[2 * i + 1], stream));
  }
  if (r->timing) {
    GB_CUDA(cudaStreamSynchronize(stream));
    for (int i = 0; i < r->n_ops; ++i) {
      const long long label = ops[i].a[23];
      float ms = 0.f;
      if (label >= 0 && label < r->n_labels && cudaEventElapsedTime(&ms, events[2 * i], events[2 * i + 1]) == cudaSuccess) {
        r->label_ms[label] += ms;
        r->label_count[label] += 1;
      }
    }
  }
  if (w.lazy_norm != nullptr) {
    snprintf(gb_error_buffer(), 512, "gb_plan_run: a norm was left to a product that never came");
    r->failed_lib = 2;
    return GB_ERR_ARG;
  }
  return w.launches;
}
