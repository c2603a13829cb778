/*
 * Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in tejkas/tinyserve-llm: it exists for hosts that embed the
 * kernel library without an allocator they may call at step time.  Examples: a serving process
 * that has already handed every free byte of the device to its own pools (as this engine does when
 * it sizes its cache from free memory), a plain C or C++ host that links the library without
 * torch, or a latency-critical loop in which cudaMalloc and cudaFree are unwelcome because they
 * synchronise the device.  ts_paged_attention_bf16 asks such a caller for a scratch buffer of
 * ts_attention_bf16_scratch_floats() floats; this variant brings its own.
 *
 * The scratch lives in a fixed array in device memory that is part of the library image, so every
 * GPU that loads the library holds TS_NOALLOC_SCRATCH_FLOATS * 4 bytes (16 MiB) until the process
 * exits.  A call whose requests, heads and context length need more than that is refused with an
 * error (ts_last_error() names the need and the limit); nothing is launched then.
 *
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and keeps it.  Make that first call on each device once at start-up,
 *    outside any stream capture.  The address is good for as long as the device's context lives:
 *    a host that tears the context down (cudaDeviceReset) must not call this again afterwards in
 *    the same process.
 *  - The function itself calls no cudaMalloc, cudaFree or other allocating routine.
 *  - All calls on a device share the one array.  Its contents are whatever the last call left; the
 *    kernels write every partial result they later read, so nothing has to be cleared between
 *    calls.  Two calls that overlap on the GPU (different streams without an ordering between
 *    them) race on the array: order them.
 *
 * Arguments are those of ts_paged_attention_bf16 for a step in which every request feeds exactly
 * one token (cu_q = 0, 1, 2, ...), without the scratch pointer.  Returns 0 on success.
 */
#pragma once

#include <cuda_runtime.h>

#define TS_NOALLOC_SCRATCH_FLOATS (4ll * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

/* Floats the built-in scratch holds (TS_NOALLOC_SCRATCH_FLOATS): compare with
 * ts_attention_bf16_scratch_floats(requests, heads, head size, longest context) before relying on this entry point. */
long long ts_decode_attention_noalloc_max_floats(void);

int ts_decode_attention_bf16_noalloc(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                                     long long page_stride, long long entry_offset, int page_tokens, int num_pages,
                                     const int* block_table, int table_width, const int* cu_q, const int* ctx_lens,
                                     int num_seqs, int max_ctx_len, int nh, int nkv, int hd, float scale, int window,
                                     cudaStream_t stream);

#ifdef __cplusplus
}
#endif
