// RMSNorm with the residual add fused in.
//
// Reference formulas (model/llama.py:52-67): s = f32(x) + f32(residual); residual' = round(s);
// y = s * rsqrt(mean(s^2) + eps) from the unrounded sum; out = round(y) * weight, rounded again.
// `rows` (optional) picks the rows to normalise, output compact: the final norm of the wanted rows.
// `gather` (optional) makes x a table whose row gather[r] is the input of row r: the token embedding
// (model/llama.py:264, 271) read straight into the model's first norm, the row itself written out as
// the start of the residual stream; an id outside the table reads as a row of zeros.
#include "common.cuh"

// Vector width in elements of a 16-byte access.
template <typename T>
struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename T, typename W, bool VECTOR>
__global__ void add_rmsnorm_kernel(const T* x, const T* residual, const W* __restrict__ weight,
                                   T* out, T* residual_out, const int* __restrict__ rows, int hidden, float eps,
                                   const int* __restrict__ gather, int gather_rows) {
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
    const int from = gather ? gather[src] : src;
    const bool zeros = gather && (from < 0 || from >= gather_rows);
    const T* xr = x + (long long)(zeros ? 0 : from) * hidden;
    const T* rr = residual ? residual + (long long)src * hidden : nullptr;
    float acc = 0.f;
    if (VECTOR) {                                  // hidden is a multiple of VN and the rows are 16-byte aligned
        for (int i = threadIdx.x * VN; i < hidden; i += blockDim.x * VN) {
            const uint4 xv = zeros ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(xr + i);
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
            float s = zeros ? 0.f : to_float<T>(xr[i]);
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

// The same for many rows (prompts): a row is held in the registers of TPR threads (up to 8 chunks of
// 16 bytes each), all its loads are in flight at once, the sum of squares goes through shuffles (and,
// for rows of more than a warp, once through shared memory), and nothing is staged in shared memory.
// 256 threads, 256 / TPR rows a CTA.  Needs 16-byte aligned rows and hidden <= TPR * 8 chunks.
template <typename T, typename W, int TPR>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(const T* x, const T* residual, const W* __restrict__ weight, T* out, T* residual_out,
                        const int* __restrict__ rows, int num_rows, int hidden, float eps, const int* __restrict__ gather,
                        int gather_rows) {
    constexpr int VN = VecOf<T>::N, MAXC = 8, RPC = 256 / TPR;
    __shared__ float part[8];
    const int group = threadIdx.x / TPR, member = threadIdx.x % TPR;
    const int r = blockIdx.x * RPC + group;
    const int chunks = hidden / VN;                       // chunk c of the row belongs to thread c % TPR
    chain_wait();
    chain_release();
    const bool live = r < num_rows;
    const int src = live ? (rows ? rows[r] : r) : -1;
    float s[MAXC][VN];
    float acc = 0.f;
    if (src >= 0) {
        const int from = gather ? gather[src] : src;
        const bool zeros = gather && (from < 0 || from >= gather_rows);
        const T* xr = x + (long long)(zeros ? 0 : from) * hidden;
        const T* rr = residual ? residual + (long long)src * hidden : nullptr;
        uint4 xv[MAXC], rv[MAXC];
#pragma unroll
        for (int k = 0; k < MAXC; ++k) {
            const int c = member + k * TPR;
            xv[k] = (c < chunks && !zeros) ? *reinterpret_cast<const uint4*>(xr + c * VN) : make_uint4(0, 0, 0, 0);
            rv[k] = (rr && c < chunks) ? *reinterpret_cast<const uint4*>(rr + c * VN) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int k = 0; k < MAXC; ++k) {
            const T* xe = reinterpret_cast<const T*>(&xv[k]);
            const T* re = reinterpret_cast<const T*>(&rv[k]);
#pragma unroll
            for (int e = 0; e < VN; ++e) {
                float v = to_float<T>(xe[e]);
                if (rr) v += to_float<T>(re[e]);
                s[k][e] = v;
                acc += v * v;
            }
        }
    }
    acc = warp_sum(acc);
    if (TPR > 32) {                                       // a row spans TPR / 32 warps: add their sums in warp order
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) part[warp] = acc;
        __syncthreads();
        acc = 0.f;
#pragma unroll
        for (int w = 0; w < TPR / 32; ++w) acc += part[group * (TPR / 32) + w];
    }
    if (src < 0) return;                                  // a padding row, or past the last row
    const float inv = rsqrtf(acc / (float)hidden + eps);
    T* outr = out + (long long)r * hidden;
    T* resr = residual_out ? residual_out + (long long)src * hidden : nullptr;
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
        const int c = member + k * TPR;
        if (c >= chunks) continue;
        uint4 ov, rv;
        T* oe = reinterpret_cast<T*>(&ov);
        T* re = reinterpret_cast<T*>(&rv);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
            re[e] = from_float<T>(s[k][e]);
            oe[e] = from_float<T>(round_to<T>(s[k][e] * inv) * to_float<W>(weight[c * VN + e]));
        }
        if (resr) *reinterpret_cast<uint4*>(resr + c * VN) = rv;
        *reinterpret_cast<uint4*>(outr + c * VN) = ov;
    }
}

template <typename T, typename W>
static int launch(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                  const int* rows, int num_rows, int hidden, float eps, const int* gather, int gather_rows,
                  cudaStream_t stream) {
    const bool vector = hidden % VecOf<T>::N == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                        (residual == nullptr || (uintptr_t)residual % 16 == 0) &&
                        (residual_out == nullptr || (uintptr_t)residual_out % 16 == 0);
    if (vector && num_rows >= 256) {                       // many rows: rows in registers, several rows a CTA
        const int chunks = hidden / VecOf<T>::N;
        const int tpr = chunks <= 32 * 8 ? 32 : (chunks <= 64 * 8 ? 64 : (chunks <= 128 * 8 ? 128 : 0));
        if (tpr != 0) {
            const int rows_per_cta = 256 / tpr;
            const dim3 grid((num_rows + rows_per_cta - 1) / rows_per_cta);
#define TS_NORM_ROWS(TPR_)                                                                                              \
    TS_CHAINED_CHECK("add_rmsnorm", launch_chained(add_rmsnorm_rows_kernel<T, W, TPR_>, grid, dim3(256), 0, stream,     \
                                                   (const T*)x, (const T*)residual, (const W*)weight, (T*)out,          \
                                                   (T*)residual_out, rows, num_rows, hidden, eps, gather, gather_rows))
            if (tpr == 32) TS_NORM_ROWS(32);
            else if (tpr == 64) TS_NORM_ROWS(64);
            else TS_NORM_ROWS(128);
#undef TS_NORM_ROWS
            return 0;
        }
    }
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
                                                   rows, hidden, eps, gather, gather_rows));
    return 0;
}

TS_API int ts_add_rmsnorm(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                          const int* rows, int num_rows, int hidden, float eps, int dtype, int weight_dtype,
                          const int* gather, int gather_rows, cudaStream_t stream) {
    TS_REQUIRE(gather == nullptr || (gather_rows > 0 && residual == nullptr && rows == nullptr),
               "add_rmsnorm: a gathered input starts the stream (no residual, no row choice) from a table with rows");
    TS_REQUIRE(num_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d H=%d", num_rows, hidden);
    TS_REQUIRE(hidden <= 56 * 1024, "add_rmsnorm: hidden size %d exceeds the kernel's limit of 57344", hidden);
    TS_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
    if (num_rows == 0) return 0;
    if (dtype == TS_F32 && weight_dtype == TS_F32)
        return launch<float, float>(x, residual, weight, out, residual_out, rows, num_rows, hidden, eps, gather, gather_rows, stream);
    if (dtype == TS_BF16 && weight_dtype == TS_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(x, residual, weight, out, residual_out, rows, num_rows, hidden, eps, gather, gather_rows, stream);
    if (dtype == TS_BF16 && weight_dtype == TS_F32)
        return launch<__nv_bfloat16, float>(x, residual, weight, out, residual_out, rows, num_rows, hidden, eps, gather, gather_rows, stream);
    return ts_fail("add_rmsnorm: unsupported dtypes activation=%d weight=%d", dtype, weight_dtype);
}
