// The error message of the last failed call on this thread (one copy per
// shared library).
#include "common.cuh"

static thread_local char g_error[512];
char* gb_error_buffer() { return g_error; }
GB_API const char* gb_last_error() { return g_error; }
