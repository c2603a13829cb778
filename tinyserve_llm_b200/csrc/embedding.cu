// Token embedding: out[t, :] = table[ids[t], :].  Reference op: nn.Embedding (model/llama.py:264,271).
#include "common.cuh"

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out,
                                 int hidden, int vocab) {
    const int t = blockIdx.x;
    chain_wait();
    chain_release();
    int id = ids[t];
    const bool valid = id >= 0 && id < vocab;      // padding rows carry id -1: they get zeros
    const T* src = table + (long long)(valid ? id : 0) * hidden;
    T* dst = out + (long long)t * hidden;
    constexpr int VN = 16 / sizeof(T);
    if (hidden % VN == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)out % 16 == 0) {
        for (int i = threadIdx.x * VN; i < hidden; i += blockDim.x * VN)
            *reinterpret_cast<uint4*>(dst + i) = valid ? *reinterpret_cast<const uint4*>(src + i) : make_uint4(0, 0, 0, 0);
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = valid ? src[i] : from_float<T>(0.f);
}

TS_API int ts_embedding(const void* table, const int* ids, void* out, int num_tokens, int hidden, int vocab,
                        int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes T=%d H=%d V=%d", num_tokens, hidden, vocab);
    if (num_tokens == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == TS_F32)
        TS_CHAINED_CHECK("embedding", launch_chained(embedding_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream,
                                                     (const float*)table, ids, (float*)out, hidden, vocab));
    else if (dtype == TS_BF16)
        TS_CHAINED_CHECK("embedding", launch_chained(embedding_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0,
                                                     stream, (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out,
                                                     hidden, vocab));
    else
        return ts_fail("embedding: unknown dtype code %d", dtype);
    return 0;
}

// A decode step launched before the host has read the previous step's samples takes its token ids
// from the sampler's output on the device: an id slot that holds -(j + 2) is replaced by src[j].
// -1 stays what it is elsewhere (a row that embeds to zeros), and so does an index out of range.
__global__ void feed_tokens_kernel(int* __restrict__ ids, int n, const int* __restrict__ src, int src_n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int v = ids[i];
    if (v < -1) {
        const int j = -v - 2;
        ids[i] = j < src_n ? src[j] : -1;
    }
}

TS_API int ts_feed_tokens(int* ids, int n, const int* src, int src_n, cudaStream_t stream) {
    TS_REQUIRE(n >= 0 && src_n >= 0, "feed_tokens: bad sizes n=%d src=%d", n, src_n);
    if (n == 0) return 0;
    feed_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, n, src, src_n);
    TS_LAUNCH_CHECK("feed_tokens");
    return 0;
}
