// Error buffer and version of the kernel library.
#include "common.cuh"

static thread_local char g_error[512] = "";

char* ts_error_buffer() { return g_error; }

TS_API const char* ts_last_error() { return g_error; }

TS_API int ts_abi_version() { return 1; }

// Programmatic dependent launch between the engine's own kernels; on by default.
static bool g_chaining = true;

bool ts_chaining_enabled() { return g_chaining; }

TS_API void ts_set_chaining(int enabled) { g_chaining = enabled != 0; }
