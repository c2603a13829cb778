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

// 16 bytes of gate and of up per thread; inter must be a multiple of the vector width.
template <typename T, int VEC>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long chunks, int inter) {
    const int per_row = inter / VEC;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < chunks;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / per_row;
        const int i = (int)(idx % per_row) * VEC;
        const T* g = gate_up + t * 2 * inter + i;
        uint4 gv = *reinterpret_cast<const uint4*>(g), uv = *reinterpret_cast<const uint4*>(g + inter), ov;
        const T* ge = reinterpret_cast<const T*>(&gv);
        const T* ue = reinterpret_cast<const T*>(&uv);
        T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float x = to_float<T>(ge[e]);
            const float silu = x / (1.f + expf(-x));
            oe[e] = from_float<T>(round_to<T>(silu) * to_float<T>(ue[e]));
        }
        *reinterpret_cast<uint4*>(out + t * inter + i) = ov;
    }
}

TS_API int ts_silu_mul(const void* gate_up, void* out, int num_tokens, int inter, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && inter > 0, "silu_mul: bad sizes T=%d I=%d", num_tokens, inter);
    if (num_tokens == 0) return 0;
    const long long total = (long long)num_tokens * inter;
    const int threads = 256;
    const int vec = dtype == TS_F32 ? 4 : 8;
    if ((dtype == TS_F32 || dtype == TS_BF16) && inter % vec == 0 && (uintptr_t)gate_up % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const long long chunks = total / vec;
        const unsigned vblocks = (unsigned)((chunks + threads - 1) / threads < 148 * 32 ? (chunks + threads - 1) / threads : 148 * 32);
        if (dtype == TS_F32)
            silu_mul_vec_kernel<float, 4><<<vblocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, chunks, inter);
        else
            silu_mul_vec_kernel<__nv_bfloat16, 8><<<vblocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                                               (__nv_bfloat16*)out, chunks, inter);
        TS_LAUNCH_CHECK("silu_mul");
        return 0;
    }
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
