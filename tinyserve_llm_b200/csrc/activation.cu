// SwiGLU gate: out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i].
// Reference (model/llama.py:80-83): silu(gate) is materialised in the activation dtype, then
// multiplied by up and rounded again; in float32 both roundings are no-ops.
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int inter) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inter;
        const int i = (int)(idx % inter);
        const float g = to_float<T>(gate_up[t * 2 * inter + i]);
        const float u = to_float<T>(gate_up[t * 2 * inter + inter + i]);
        const float silu = g / (1.f + expf(-g));
        out[idx] = from_float<T>(round_to<T>(silu) * u);
    }
}

TS_API int ts_silu_mul(const void* gate_up, void* out, int num_tokens, int inter, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && inter > 0, "silu_mul: bad sizes T=%d I=%d", num_tokens, inter);
    if (num_tokens == 0) return 0;
    const long long total = (long long)num_tokens * inter;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == TS_F32)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, total, inter);
    else if (dtype == TS_BF16)
        silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                                      (__nv_bfloat16*)out, total, inter);
    else
        return ts_fail("silu_mul: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("silu_mul");
    return 0;
}
