// RMSNorm with the residual add fused in.
//
// Reference formulas (model/llama.py:52-67): s = f32(x) + f32(residual); residual' = round(s);
// y = s * rsqrt(mean(s^2) + eps) from the unrounded sum; out = round(y) * weight, rounded again.
// `rows` (optional) picks the rows to normalise, output compact: the final norm of the wanted rows.
#include "common.cuh"

// Vector width in elements of a 16-byte access.
template <typename T>
struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename T, typename W, bool VECTOR>
__global__ void add_rmsnorm_kernel(const T* x, const T* residual, const W* __restrict__ weight,
                                   T* out, T* residual_out, const int* __restrict__ rows, int hidden, float eps) {
    extern __shared__ float sums[];              // hidden floats: the unrounded sum, then 33 of scratch
    float* scratch = sums + hidden;
    const int r = blockIdx.x;
    constexpr int VN = VecOf<T>::N;
    // the weights do not depend on the kernel ahead on the stream: the thread's first chunk is asked
    // for before the wait for that kernel
    float wv[VN];
    const int i0 = threadIdx.x * VN;
    if (VECTOR && i0 < hidden) {
#pragma unroll
        for (int e = 0; e < VN; ++e) wv[e] = to_float<W>(weight[i0 + e]);
    }
    chain_wait();
    chain_release();
    const int src = rows ? rows[r] : r;
    if (src < 0) return;                          // a padding row
    const T* xr = x + (long long)src * hidden;
    const T* rr = residual ? residual + (long long)src * hidden : nullptr;
    float acc = 0.f;
    if (VECTOR) {                                  // hidden is a multiple of VN and the rows are 16-byte aligned
        for (int i = threadIdx.x * VN; i < hidden; i += blockDim.x * VN) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xr + i);
            uint4 rv = make_uint4(0, 0, 0, 0);
            if (rr) rv = *reinterpret_cast<const uint4*>(rr + i);
            const T* xe = reinterpret_cast<const T*>(&xv);
            const T* re = reinterpret_cast<const T*>(&rv);
#pragma unroll
            for (int e = 0; e < VN; ++e) {
                float s = to_float<T>(xe[e]);
                if (rr) s += to_float<T>(re[e]);
                sums[i + e] = s;
                acc += s * s;
            }
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float s = to_float<T>(xr[i]);
            if (rr) s += to_float<T>(rr[i]);
            sums[i] = s;
            acc += s * s;
        }
    }
    const float total = block_sum(acc, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    T* outr = out + (long long)r * hidden;
    T* resr = residual_out ? residual_out + (long long)src * hidden : nullptr;
    if (VECTOR) {
        for (int i = threadIdx.x * VN; i < hidden; i += blockDim.x * VN) {
            uint4 ov, rv;
            T* oe = reinterpret_cast<T*>(&ov);
            T* re = reinterpret_cast<T*>(&rv);
#pragma unroll
            for (int e = 0; e < VN; ++e) {
                const float s = sums[i + e];
                re[e] = from_float<T>(s);
                const float w = i == i0 ? wv[e] : to_float<W>(weight[i + e]);
                oe[e] = from_float<T>(round_to<T>(s * inv) * w);
            }
            if (resr) *reinterpret_cast<uint4*>(resr + i) = rv;
            *reinterpret_cast<uint4*>(outr + i) = ov;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float s = sums[i];
            if (resr) resr[i] = from_float<T>(s);
            outr[i] = from_float<T>(round_to<T>(s * inv) * to_float<W>(weight[i]));
        }
    }
}

template <typename T, typename W>
static int launch(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                  const int* rows, int num_rows, int hidden, float eps, cudaStream_t stream) {
    const bool vector = hidden % VecOf<T>::N == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                        (residual == nullptr || (uintptr_t)residual % 16 == 0) &&
                        (residual_out == nullptr || (uintptr_t)residual_out % 16 == 0);
    const int per_thread = vector ? VecOf<T>::N : 1;
    int threads = 128;
    while (threads < 512 && threads * per_thread < hidden) threads *= 2;
    const size_t smem = (size_t)(hidden + 33) * sizeof(float);
    auto kernel = vector ? add_rmsnorm_kernel<T, W, true> : add_rmsnorm_kernel<T, W, false>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ts_fail("add_rmsnorm: cannot reserve %zu bytes of shared memory: %s", smem,
                                             cudaGetErrorString(e));
    }
    TS_CHAINED_CHECK("add_rmsnorm", launch_chained(kernel, dim3(num_rows), dim3(threads), smem, stream, (const T*)x,
                                                   (const T*)residual, (const W*)weight, (T*)out, (T*)residual_out,
                                                   rows, hidden, eps));
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
