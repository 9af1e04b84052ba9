// What a kernel library outside this package needs in order to add an operation to the step
// plan (csrc/step_plan.cu): the signature of the operation's function, what it sees of a step,
// and the order of the step's symbols.
//
// A part with kernels of its own exports one function per operation,
//
//     extern "C" int my_op(const GbPlanCtx* ctx, const long long* a, const double* f, int flags);
//
// registers it under a name (Python: gibbs_b200.engine.plan.register_op(name, function); C:
// gb_plan_register_op) and emits records with the id it got back (PlanBuilder.emit(id, a, f,
// flags)).  When a step reaches the record, the function is called with the record's 24 integer
// operands (an operand that named a symbol holds the step's value of it: a count, or a device
// address), its 3 floating-point operands and its flags.  It launches its kernels on
// ctx->stream and returns how many it launched, or a negative number to fail the step.
// Before the call the 32-bit residual stream is whole (sums that a product had left to be added
// are added).
#pragma once
#include <cuda_runtime.h>

struct GbPlanCtx {
  cudaStream_t stream;
  int* status;               // the device's status word (a kernel sets it nonzero to report a failure)
  const long long* sym;      // the step's symbols, indexed by GbPlanSymbol
  int n_sym;
};

typedef int (*GbPlanOpFn)(const GbPlanCtx* ctx, const long long* a, const double* f, int flags);

// Counts are values; the rest are device addresses of int32 arrays of the step's metadata.
enum GbPlanSymbol : int {
  GB_SYM_TOKENS = 0,         // tokens in the step
  GB_SYM_REQUESTS,           // requests in the step
  GB_SYM_WANTED,             // rows whose logits are wanted
  GB_SYM_MAX_PORTION,        // longest portion of the step
  GB_SYM_MAX_CONTEXT,        // longest context after the step (an upper bound inside CUDA graphs)
  GB_SYM_ONE_EACH,           // 1 when every request brings exactly one token
  GB_SYM_TOKEN_IDS,          // [tokens]
  GB_SYM_TOKEN_REQUEST,      // [tokens] index of the token's request within the step
  GB_SYM_TOKEN_POSITION,     // [tokens] position of the token in its request
  GB_SYM_PORTION_START,      // [requests] row of the request's first token
  GB_SYM_PORTION_LENGTH,     // [requests]
  GB_SYM_LENGTH_BEFORE,      // [requests] the request's length before the step
  GB_SYM_LENGTH_AFTER,       // [requests]
  GB_SYM_SLOT_IDS,           // [requests] state slot of the request
  GB_SYM_WANTED_ROWS,        // [wanted]
  GB_SYM_LOGITS,             // float32 [wanted, vocabulary]
  GB_SYM_BLOCK_TABLE0,       // + g (g < 15): block table of cache group g, [requests, GB_SYM_TABLE_STRIDE entries]
  GB_SYM_TABLE_STRIDE = 31,  // entries per request in this step's block tables (a value)
  GB_SYM_COUNT = 32
};
