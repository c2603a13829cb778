// RMSNorm with the residual add fused in.
//
// Reference formulas (model/llama.py:52-67): s = f32(x) + f32(residual); residual' = round(s);
// y = s * rsqrt(mean(s^2) + eps) from the unrounded sum; out = round(y) * weight, rounded again.
// `rows` (optional) picks the rows to normalise, output compact: the final norm of the wanted rows.
#include "common.cuh"

template <typename T, typename W>
__global__ void add_rmsnorm_kernel(const T* x, const T* residual, const W* __restrict__ weight,
                                   T* out, T* residual_out, const int* __restrict__ rows, int hidden, float eps) {
    extern __shared__ float sums[];              // hidden floats: the unrounded sum, then 33 of scratch
    float* scratch = sums + hidden;
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    if (src < 0) return;                          // a padding row
    const T* xr = x + (long long)src * hidden;
    const T* rr = residual ? residual + (long long)src * hidden : nullptr;
    float acc = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float s = to_float<T>(xr[i]);
        if (rr) s += to_float<T>(rr[i]);
        sums[i] = s;
        acc += s * s;
    }
    const float total = block_sum(acc, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    T* outr = out + (long long)r * hidden;
    T* resr = residual_out ? residual_out + (long long)src * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float s = sums[i];
        if (resr) resr[i] = from_float<T>(s);
        outr[i] = from_float<T>(round_to<T>(s * inv) * to_float<W>(weight[i]));
    }
}

template <typename T, typename W>
static int launch(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                  const int* rows, int num_rows, int hidden, float eps, cudaStream_t stream) {
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const size_t smem = (size_t)(hidden + 33) * sizeof(float);
    auto kernel = add_rmsnorm_kernel<T, W>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ts_fail("add_rmsnorm: cannot reserve %zu bytes of shared memory: %s", smem,
                                             cudaGetErrorString(e));
    }
    kernel<<<num_rows, threads, smem, stream>>>((const T*)x, (const T*)residual, (const W*)weight, (T*)out,
                                                (T*)residual_out, rows, hidden, eps);
    TS_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

TS_API int ts_add_rmsnorm(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                          const int* rows, int num_rows, int hidden, float eps, int dtype, int weight_dtype,
                          cudaStream_t stream) {
    TS_REQUIRE(num_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d H=%d", num_rows, hidden);
    TS_REQUIRE(hidden <= 56 * 1024, "add_rmsnorm: hidden size %d exceeds the kernel's limit of 57344", hidden);
    TS_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
    if (num_rows == 0) return 0;
    if (dtype == TS_F32 && weight_dtype == TS_F32)
        return launch<float, float>(x, residual, weight, out, residual_out, rows, num_rows, hidden, eps, stream);
    if (dtype == TS_BF16 && weight_dtype == TS_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(x, residual, weight, out, residual_out, rows, num_rows, hidden, eps, stream);
    if (dtype == TS_BF16 && weight_dtype == TS_F32)
        return launch<__nv_bfloat16, float>(x, residual, weight, out, residual_out, rows, num_rows, hidden, eps, stream);
    return ts_fail("add_rmsnorm: unsupported dtypes activation=%d weight=%d", dtype, weight_dtype);
}
