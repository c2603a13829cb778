// Copy of the first n token slots of one cache page to another, for every entry and kv head of a
// layer group, keys and values: copy-on-write of a shared last page and reuse of a partly matching
// cached page.  Reference op: KVStorage.copy_slots (kvcache/storage.py:43-50).
#include "common.cuh"

__global__ void copy_page_slots_kernel(uint4* k_pool, uint4* v_pool, long long page_stride16, long long run_stride16,
                                       int runs, int src, int dst, long long copy16) {
    uint4* pool = blockIdx.y == 0 ? k_pool : v_pool;
    const int run = blockIdx.x;                               // one (entry, kv head) stretch of the page
    if (run >= runs) return;
    const uint4* s = pool + (long long)src * page_stride16 + (long long)run * run_stride16;
    uint4* d = pool + (long long)dst * page_stride16 + (long long)run * run_stride16;
    for (long long i = threadIdx.x; i < copy16; i += blockDim.x) d[i] = s[i];
}

TS_API int ts_copy_page_slots(void* k_pool, void* v_pool, int num_pages, int entries, int nkv, int page_tokens, int hd,
                              int elem_bytes, int src_page, int dst_page, int num_slots, cudaStream_t stream) {
    TS_REQUIRE(src_page >= 0 && src_page < num_pages && dst_page >= 0 && dst_page < num_pages,
               "copy_page_slots: pages %d -> %d outside the pool of %d", src_page, dst_page, num_pages);
    TS_REQUIRE(num_slots >= 0 && num_slots <= page_tokens, "copy_page_slots: %d slots of a %d-token page", num_slots, page_tokens);
    TS_REQUIRE(((long long)hd * elem_bytes) % 16 == 0, "copy_page_slots: a head row of %d bytes is not a multiple of 16",
               hd * elem_bytes);
    if (num_slots == 0 || src_page == dst_page) return 0;
    const long long run16 = (long long)page_tokens * hd * elem_bytes / 16;
    const long long page16 = run16 * entries * nkv;
    const long long copy16 = (long long)num_slots * hd * elem_bytes / 16;
    dim3 grid(entries * nkv, 2);
    copy_page_slots_kernel<<<grid, 128, 0, stream>>>((uint4*)k_pool, (uint4*)v_pool, page16, run16, entries * nkv,
                                                    src_page, dst_page, copy16);
    TS_LAUNCH_CHECK("copy_page_slots");
    return 0;
}
