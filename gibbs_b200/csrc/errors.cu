// The error message of the last failed call on this thread (one copy per
// shared library).
#include "common.cuh"

static thread_local char g_error[512];
char* gb_error_buffer() { return g_error; }
GB_API const char* gb_last_error() { return g_error; }

#include <stdlib.h>
int gb_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("GIBBS_B200_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v;
}
