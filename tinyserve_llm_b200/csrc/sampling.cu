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

// (value, index) with the greater value, ties to the lower index; index 0x7fffffff marks "nothing yet".
struct Best {
    float v;
    int i;
};
constexpr int NOTHING = 0x7fffffff;

__device__ __forceinline__ void take(Best& b, float v, int i) {
    if (i != NOTHING && (b.i == NOTHING || v > b.v || (v == b.v && i < b.i))) {
        b.v = v;
        b.i = i;
    }
}

// The best of the block in thread 0.
__device__ __forceinline__ Best block_best(Best b, float* best_v, int* best_i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        take(b, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = b.v; best_i[warp] = b.i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int nwarps = (blockDim.x + 31) >> 5;
        for (int w = 1; w < nwarps; ++w) take(b, best_v[w], best_i[w]);
    }
    return b;
}

__device__ __forceinline__ float noisy(float v, int i, float temp, uint32_t k0, uint32_t k1) {
    const uint32_t bits = philox_first_word((uint32_t)i, 0u, k0, k1);
    // 23 bits, so that u + 0.5 ulp is still a float32 below 1: with 24 bits the largest value rounded to 1.0,
    // whose noise is +infinity, and one logit in 2^24 was drawn whatever its value
    const float u = ((float)(bits >> 9) + 0.5f) * (1.0f / 8388608.0f);    // in (0, 1), both ends excluded
    const float e = -logf(u);                                              // Exp(1), > 0
    return v / temp - logf(e);
}

// A row is cut into chunks of SAMPLE_CHUNK logits, one CTA each, so that a few rows of a large
// vocabulary still keep many SMs loading; a second kernel picks the best chunk of each row.  The
// result does not depend on the cut: the maximum is the maximum, ties go to the lowest index.
constexpr int SAMPLE_THREADS = 256, SAMPLE_CHUNK = SAMPLE_THREADS * 16;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_chunk_kernel(const float* __restrict__ logits, long long row_stride, const float* __restrict__ temperatures,
                    const uint32_t* __restrict__ keys, float* __restrict__ part_v, int* __restrict__ part_i, int vocab,
                    int chunks, int vector) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int r = blockIdx.y, chunk = blockIdx.x;
    const float temp = temperatures[r];                    // written by the host before the step
    const uint32_t k0 = keys[2 * r], k1 = keys[2 * r + 1];
    chain_wait();
    chain_release();
    const float* row = logits + (long long)r * row_stride;
    const int base = chunk * SAMPLE_CHUNK;
    Best b{-INFINITY, NOTHING};
    if (vector) {                                          // rows start 16-byte aligned and the vocabulary is a multiple of 4
        float4 v[4];
        int at[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {                      // all four loads before any is used
            at[k] = base + (k * SAMPLE_THREADS + threadIdx.x) * 4;
            v[k] = at[k] < vocab ? *reinterpret_cast<const float4*>(row + at[k]) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (at[k] >= vocab) continue;
            float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (temp > 0.f) e[j] = noisy(e[j], at[k] + j, temp, k0, k1);
                take(b, e[j], at[k] + j);
            }
        }
    } else {
        for (int i = base + threadIdx.x; i < min(vocab, base + SAMPLE_CHUNK); i += SAMPLE_THREADS) {
            float v = row[i];
            if (temp > 0.f) v = noisy(v, i, temp, k0, k1);
            take(b, v, i);
        }
    }
    b = block_best(b, best_v, best_i);
    if (threadIdx.x == 0) {
        part_v[(long long)r * chunks + chunk] = b.v;
        part_i[(long long)r * chunks + chunk] = b.i;
    }
}

__global__ void sample_pick_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int* __restrict__ out,
                                   int chunks) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int r = blockIdx.x;
    chain_wait();
    chain_release();
    Best b{-INFINITY, NOTHING};
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) take(b, part_v[(long long)r * chunks + c], part_i[(long long)r * chunks + c]);
    b = block_best(b, best_v, best_i);
    if (threadIdx.x == 0) out[r] = b.i == NOTHING ? 0 : b.i;
}

TS_API int ts_sample_scratch_words(int num_rows, int vocab) {
    return 2 * num_rows * ((vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK);
}

// scratch: ts_sample_scratch_words(num_rows, vocab) 32-bit words on the device.
TS_API int ts_sample(const float* logits, long long row_stride, const float* temperatures, const uint32_t* keys,
                     int* out, int num_rows, int vocab, void* scratch, int scratch_words, cudaStream_t stream) {
    TS_REQUIRE(num_rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d V=%d", num_rows, vocab);
    if (num_rows == 0) return 0;
    TS_REQUIRE(num_rows <= 65535, "sample: more than 65535 rows in a call");
    const int chunks = (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    TS_REQUIRE(scratch != nullptr && scratch_words >= 2 * num_rows * chunks, "sample: scratch of %d words is too small", scratch_words);
    float* part_v = (float*)scratch;
    int* part_i = (int*)scratch + (long long)num_rows * chunks;
    const int vector = vocab % 4 == 0 && row_stride % 4 == 0 && (uintptr_t)logits % 16 == 0;
    TS_CHAINED_CHECK("sample", launch_chained(sample_chunk_kernel, dim3(chunks, num_rows), dim3(SAMPLE_THREADS), 0, stream,
                                              logits, row_stride, temperatures, keys, part_v, part_i, vocab, chunks, vector));
    TS_CHAINED_CHECK("sample", launch_chained(sample_pick_kernel, dim3(num_rows), dim3(128), 0, stream, (const float*)part_v,
                                              (const int*)part_i, out, chunks));
    return 0;
}
