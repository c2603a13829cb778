// Paged causal grouped-query attention, generic version: any head size that is a multiple of 16 up
// to 256, any number of heads and groups, any page size, float32 or bfloat16 storage.  One kernel
// serves whole prompts, portions of prompts over a cached prefix, and single decoded tokens: the
// step's keys are in the cache before it runs, and a query at position p sees keys max(0, p-w+1)..p
// (w = window, 0 for all), which is the bottom-right-aligned causal rule of
// attention/torch_paged.py:36-45 (reference) expressed through positions.
//
// One warp per (token, query head).  Lane l takes keys lo+l, lo+l+32, ... and keeps its own running
// maximum, sum and output; lanes merge at the end.  The order of every sum depends only on the
// query's position, never on how the step was cut or what else is in the batch.  Softmax and both
// products accumulate in float32.
#include "common.cuh"

template <typename T>
struct Vec16;   // 16 bytes of T
template <>
struct Vec16<float> { static constexpr int N = 4; };
template <>
struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&out)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
}

constexpr int WARPS = 4;

template <typename T, int MAXHD>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ qkv, T* __restrict__ out, const T* __restrict__ k_pool,
                               const T* __restrict__ v_pool, KVGeometry geo, const int* __restrict__ block_table,
                               int table_width, const int* __restrict__ positions,
                               const int* __restrict__ seq_of_token, int num_tokens, int nh, int nkv, int hd,
                               float scale, int window) {
    __shared__ float q_smem[WARPS][MAXHD];
    constexpr int VN = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)num_tokens * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    const int seq = seq_of_token[t];
    T* o_ptr = out + ((long long)t * nh + h) * hd;
    if (seq < 0) return;                                      // padding row
    const int pos = positions[t];
    const int kvh = h / (nh / nkv);
    const int row_width = (nh + 2 * nkv) * hd;
    const T* q_ptr = qkv + (long long)t * row_width + (long long)h * hd;
    for (int d = lane; d < hd; d += 32) q_smem[warp][d] = to_float<T>(q_ptr[d]) * scale;
    __syncwarp();

    float o[MAXHD];
#pragma unroll
    for (int d = 0; d < MAXHD; ++d) o[d] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const long long head_off = geo.entry_offset + (long long)kvh * geo.page_tokens * hd;
    const int* table = block_table + (long long)seq * table_width;
    for (int j = lo + lane; j <= pos; j += 32) {
        const int page = table[j / geo.page_tokens];
        if (page < 0 || page >= geo.num_pages) continue;      // a page given back (window) or a bad table
        const long long off = (long long)page * geo.page_stride + head_off + (long long)(j % geo.page_tokens) * hd;
        const T* kp = k_pool + off;
        float s = 0.f;
#pragma unroll
        for (int d0 = 0; d0 < MAXHD; d0 += VN) {
            if (d0 < hd) {
                float kv[VN];
                load16<T>(kp + d0, kv);
#pragma unroll
                for (int e = 0; e < VN; ++e) s = fmaf(q_smem[warp][d0 + e], kv[e], s);
            }
        }
        if (s > m) {
            const float c = expf(m - s);                       // 0 on the first key (m = -inf)
            l *= c;
#pragma unroll
            for (int d = 0; d < MAXHD; ++d) o[d] *= c;
            m = s;
        }
        const float p = expf(s - m);
        l += p;
        const T* vp = v_pool + off;
#pragma unroll
        for (int d0 = 0; d0 < MAXHD; d0 += VN) {
            if (d0 < hd) {
                float vv[VN];
                load16<T>(vp + d0, vv);
#pragma unroll
                for (int e = 0; e < VN; ++e) o[d0 + e] = fmaf(p, vv[e], o[d0 + e]);
            }
        }
    }
    // merge the lanes
    const float m_all = warp_max(m);
    const float f = (m == -INFINITY) ? 0.f : expf(m - m_all);
    const float l_all = warp_sum(l * f);
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
#pragma unroll
    for (int d = 0; d < MAXHD; ++d) {
        if (d < hd) {
            const float total = warp_sum(o[d] * f);
            if (lane == (d & 31)) o_ptr[d] = from_float<T>(total * inv);
        }
    }
}

template <typename T, int MAXHD>
static int launch(const void* qkv, void* out, const void* k_pool, const void* v_pool, KVGeometry geo,
                  const int* block_table, int table_width, const int* positions, const int* seq_of_token,
                  int num_tokens, int nh, int nkv, int hd, float scale, int window, cudaStream_t stream) {
    const long long items = (long long)num_tokens * nh;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    paged_attention_generic_kernel<T, MAXHD><<<blocks, WARPS * 32, 0, stream>>>(
        (const T*)qkv, (T*)out, (const T*)k_pool, (const T*)v_pool, geo, block_table, table_width, positions,
        seq_of_token, num_tokens, nh, nkv, hd, scale, window);
    TS_LAUNCH_CHECK("paged_attention_generic");
    return 0;
}

TS_API int ts_paged_attention_generic(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                                      long long page_stride, long long entry_offset, int page_tokens, int num_pages,
                                      const int* block_table, int table_width, const int* positions,
                                      const int* seq_of_token, int num_tokens, int nh, int nkv, int hd, float scale,
                                      int window, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && nh > 0 && nkv > 0, "paged_attention: bad sizes");
    TS_REQUIRE(nh % nkv == 0, "paged_attention: %d query heads are not a multiple of %d kv heads", nh, nkv);
    TS_REQUIRE(hd > 0 && hd % 16 == 0 && hd <= 256,
               "paged_attention: head_dim %d is not supported (multiples of 16 up to 256)", hd);
    TS_REQUIRE(page_tokens > 0 && table_width > 0 && window >= 0, "paged_attention: bad page geometry");
    if (num_tokens == 0) return 0;
    KVGeometry geo{page_stride, entry_offset, page_tokens, num_pages};
#define TS_DISPATCH(TYPE)                                                                                          \
    if (hd <= 32) return launch<TYPE, 32>(qkv, out, k_pool, v_pool, geo, block_table, table_width, positions,       \
                                          seq_of_token, num_tokens, nh, nkv, hd, scale, window, stream);             \
    if (hd <= 64) return launch<TYPE, 64>(qkv, out, k_pool, v_pool, geo, block_table, table_width, positions,       \
                                          seq_of_token, num_tokens, nh, nkv, hd, scale, window, stream);             \
    if (hd <= 128) return launch<TYPE, 128>(qkv, out, k_pool, v_pool, geo, block_table, table_width, positions,     \
                                            seq_of_token, num_tokens, nh, nkv, hd, scale, window, stream);           \
    return launch<TYPE, 256>(qkv, out, k_pool, v_pool, geo, block_table, table_width, positions, seq_of_token,      \
                             num_tokens, nh, nkv, hd, scale, window, stream);
    if (dtype == TS_F32) { TS_DISPATCH(float) }
    if (dtype == TS_BF16) { TS_DISPATCH(__nv_bfloat16) }
#undef TS_DISPATCH
    return ts_fail("paged_attention: unknown dtype code %d", dtype);
}
