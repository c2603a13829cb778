// Error buffer and version of the kernel library.
#include "common.cuh"

static thread_local char g_error[512] = "";

char* ts_error_buffer() { return g_error; }

TS_API const char* ts_last_error() { return g_error; }

TS_API int ts_abi_version() { return 1; }
