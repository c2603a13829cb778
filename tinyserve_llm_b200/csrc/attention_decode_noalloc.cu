// Decode attention with built-in scratch, for callers that cannot allocate device memory.
// The contract is in attention_decode_noalloc.h.  The work is done by the same kernels as
// ts_paged_attention_bf16 (attention_bf16.cu); this file only supplies their scratch.
#include "attention_decode_noalloc.h"

#include <mutex>

#include "attention_bf16.h"
#include "common.cuh"

// Partial outputs and (max, sum) pairs of the decode splits.  In host code this name is only a
// handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_decode_scratch[TS_NOALLOC_SCRATCH_FLOATS];

namespace {

constexpr int MAX_DEVICES = 64;
std::mutex g_lock;
float* g_scratch_address[MAX_DEVICES] = {};

// Device address of the scratch array on the current device, looked up once per device.
int scratch_on_current_device(float** address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return ts_fail("decode_attention_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (device < 0 || device >= MAX_DEVICES) return ts_fail("decode_attention_noalloc: device %d is out of range", device);
    std::lock_guard<std::mutex> guard(g_lock);
    if (g_scratch_address[device] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess || p == nullptr)
            return ts_fail("decode_attention_noalloc: cudaGetSymbolAddress failed on device %d: %s", device,
                           cudaGetErrorString(e));
        g_scratch_address[device] = static_cast<float*>(p);
    }
    *address = g_scratch_address[device];
    return 0;
}

}  // namespace

TS_API long long ts_decode_attention_noalloc_max_floats() { return TS_NOALLOC_SCRATCH_FLOATS; }

TS_API int ts_decode_attention_bf16_noalloc(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                                            long long page_stride, long long entry_offset, int page_tokens,
                                            int num_pages, const int* block_table, int table_width, const int* cu_q,
                                            const int* ctx_lens, int num_seqs, int max_ctx_len, int nh, int nkv, int hd,
                                            float scale, int window, cudaStream_t stream) {
    TS_REQUIRE(num_seqs >= 0 && max_ctx_len >= 0 && nh > 0 && hd > 0, "decode_attention_noalloc: bad sizes");
    const long long need = ts_attention_bf16_scratch_floats(num_seqs, nh, hd, max_ctx_len);
    TS_REQUIRE(need <= TS_NOALLOC_SCRATCH_FLOATS,
               "decode_attention_noalloc: %d requests x %d heads x context %d need %lld floats of scratch; the built-in "
               "scratch holds %lld (use ts_paged_attention_bf16 with a buffer of your own)",
               num_seqs, nh, max_ctx_len, need, (long long)TS_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (scratch_on_current_device(&scratch) != 0) return 1;
    return ts_paged_attention_bf16(qkv, out, k_pool, v_pool, page_stride, entry_offset, page_tokens, num_pages,
                                   block_table, table_width, cu_q, ctx_lens, num_seqs, /*max_q_len=*/1, /*min_q_len=*/1,
                                   max_ctx_len, nh, nkv, hd, scale, window, scratch, TS_NOALLOC_SCRATCH_FLOATS, nullptr, 0, stream);
}
