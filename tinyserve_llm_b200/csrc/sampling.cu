// Sampling of one token per logits row: greedy (temperature 0) or a draw from softmax(logits / T).
//
// Reference (engine/sampler.py:13-23): greedy = argmax; otherwise argmax(softmax(l / T) / E) with
// E ~ Exp(1), the Gumbel-max trick in exponential form.  argmax(p_i / E_i) = argmax(l_i / T - log E_i),
// so no softmax is formed.  The noise is counter-based (Philox 4x32, 10 rounds) with a key per row,
// so a request's draws do not depend on what else is in the batch.  Ties go to the lowest index.
#include "common.cuh"

__device__ __forceinline__ uint32_t mulhi32(uint32_t a, uint32_t b) { return __umulhi(a, b); }

__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
    uint32_t c2 = 0, c3 = 0;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = mulhi32(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = mulhi32(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c0;
}

__global__ void sample_kernel(const float* __restrict__ logits, long long row_stride,
                              const float* __restrict__ temperatures, const uint32_t* __restrict__ keys,
                              int* __restrict__ out, int vocab) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int r = blockIdx.x;
    chain_wait();
    chain_release();
    const float* row = logits + (long long)r * row_stride;
    const float temp = temperatures[r];
    const uint32_t k0 = keys[2 * r], k1 = keys[2 * r + 1];
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = row[i];
        if (temp > 0.f) {
            const uint32_t bits = philox_first_word((uint32_t)i, 0u, k0, k1);
            const float u = ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);   // in (0, 1)
            const float e = -logf(u);                                              // Exp(1), > 0
            v = v / temp - logf(e);
        }
        if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { bv = v; bi = i; }
    }
    // the best of the warp, then of the block; ties to the lowest index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int nwarps = (blockDim.x + 31) >> 5;
        for (int w = 1; w < nwarps; ++w) {
            const float ov = best_v[w];
            const int oi = best_i[w];
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        out[r] = bi == 0x7fffffff ? 0 : bi;
    }
}

TS_API int ts_sample(const float* logits, long long row_stride, const float* temperatures, const uint32_t* keys,
                     int* out, int num_rows, int vocab, cudaStream_t stream) {
    TS_REQUIRE(num_rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d V=%d", num_rows, vocab);
    if (num_rows == 0) return 0;
    const int threads = vocab >= 4096 ? 1024 : 256;
    TS_CHAINED_CHECK("sample", launch_chained(sample_kernel, dim3(num_rows), dim3(threads), 0, stream, logits, row_stride,
                                              temperatures, keys, out, vocab));
    return 0;
}
