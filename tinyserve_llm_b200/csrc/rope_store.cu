// Rotary position encoding of q and k fused with the write of k and v into the paged cache.
//
// Reference: rotate-half with float32 cos/sin gathered by position (model/llama.py:131-136,163-169);
// keys are stored rotated, values raw, at the slot the block table gives the token's position
// (engine/model_runner.py:60,100-102; attention/flash_backend.py:22-55).
//
// qkv is [T, (nh + 2 nkv) * hd], columns [q | k | v]; q is rotated in place, k and v go to the pool.
// `table` is [table_rows, rot] float32, cos of the rot/2 angles then their sin; dims >= rot pass
// through unrotated; a null table stores k unrotated (position applied elsewhere, or none).
#include "common.cuh"

template <typename T>
__global__ void rope_store_kernel(T* qkv, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                  const float* __restrict__ table, int rot, const int* __restrict__ block_table,
                                  int table_width, T* k_pool, T* v_pool, KVGeometry geo, int nh, int nkv, int hd,
                                  int write_kv) {
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;                                     // padding row
    const int pos = positions[t];
    const int row_width = (nh + 2 * nkv) * hd;
    T* row = qkv + (long long)t * row_width;
    const float* cs = table ? table + (long long)pos * rot : nullptr;
    const int half = rot / 2;

    long long base = -1;
    if (write_kv) {
        const int page = block_table[(long long)seq * table_width + pos / geo.page_tokens];
        if (page >= 0 && page < geo.num_pages)
            base = (long long)page * geo.page_stride + geo.entry_offset + (long long)(pos % geo.page_tokens) * hd;
    }
    const long long head_stride = (long long)geo.page_tokens * hd;

    // q and k heads: one thread per (head, pair index or pass-through dim)
    const int per_head = hd - half;                          // half pairs + (hd - rot) untouched dims
    const int rotated_heads = nh + nkv;
    for (int w = threadIdx.x; w < rotated_heads * per_head; w += blockDim.x) {
        const int head = w / per_head, i = w % per_head;
        T* h = row + (long long)head * hd;
        const bool is_k = head >= nh;
        T* dst = (is_k && base >= 0) ? k_pool + base + (long long)(head - nh) * head_stride : nullptr;
        if (i < half) {
            const float x1 = to_float<T>(h[i]), x2 = to_float<T>(h[i + half]);
            float y1 = x1, y2 = x2;
            if (cs) {
                const float c = cs[i], s = cs[half + i];
                y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));       // every product rounded, as the reference does
                y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
            }
            const T o1 = from_float<T>(y1), o2 = from_float<T>(y2);
            if (!is_k) { h[i] = o1; h[i + half] = o2; }
            else if (dst) { dst[i] = o1; dst[i + half] = o2; }
        } else {
            const int d = rot + (i - half);                  // dims past the rotary part
            if (is_k && dst) dst[d] = h[d];
        }
    }
    if (base >= 0) {
        const T* v = row + (long long)(nh + nkv) * hd;
        for (int w = threadIdx.x; w < nkv * hd; w += blockDim.x) {
            const int head = w / hd, d = w % hd;
            v_pool[base + (long long)head * head_stride + d] = v[w];
        }
    }
}

// The same with 16-byte accesses: a thread rotates VN dims of the first half against their partners.
// Needs rot / 2 and hd to be multiples of VN and 16-byte aligned rows.
template <typename T, int VN>
__global__ void rope_store_vec_kernel(T* qkv, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                      const float* __restrict__ table, int rot, const int* __restrict__ block_table,
                                      int table_width, T* k_pool, T* v_pool, KVGeometry geo, int nh, int nkv, int hd,
                                      int write_kv) {
    const int t = blockIdx.x;
    // Before the wait for the kernel ahead on the stream (the q/k/v projection): the index data,
    // which the host wrote before the step, and the angles of the thread's first chunk.
    const int seq = seq_of_token[t];
    if (seq < 0) {
        chain_wait();
        chain_release();
        return;
    }
    const int pos = positions[t];
    const int row_width = (nh + 2 * nkv) * hd;
    T* row = qkv + (long long)t * row_width;
    const float* cs = table ? table + (long long)pos * rot : nullptr;
    const int half = rot / 2;
    long long base = -1;
    if (write_kv) {
        const int page = block_table[(long long)seq * table_width + pos / geo.page_tokens];
        if (page >= 0 && page < geo.num_pages)
            base = (long long)page * geo.page_stride + geo.entry_offset + (long long)(pos % geo.page_tokens) * hd;
    }
    const long long head_stride = (long long)geo.page_tokens * hd;
    const int pair_chunks = half / VN, pass_chunks = (hd - rot) / VN;
    const int per_head = pair_chunks + pass_chunks;
    const int total = (nh + nkv) * per_head;
    float c[VN], sn[VN];
    auto load_angles = [&](int i) {
#pragma unroll
        for (int e = 0; e < VN; e += 4) {
            const float4 cv = *reinterpret_cast<const float4*>(cs + i + e);
            const float4 sv = *reinterpret_cast<const float4*>(cs + half + i + e);
            c[e] = cv.x, c[e + 1] = cv.y, c[e + 2] = cv.z, c[e + 3] = cv.w;
            sn[e] = sv.x, sn[e + 1] = sv.y, sn[e + 2] = sv.z, sn[e + 3] = sv.w;
        }
    };
    bool have_angles = false;
    if (cs && (int)threadIdx.x < total && (int)threadIdx.x % per_head < pair_chunks) {
        load_angles(((int)threadIdx.x % per_head) * VN);
        have_angles = true;
    }
    chain_wait();
    chain_release();
    for (int w = threadIdx.x; w < total; w += blockDim.x) {
        const int head = w / per_head, ch = w % per_head;
        T* h = row + (long long)head * hd;
        const bool is_k = head >= nh;
        T* dst = (is_k && base >= 0) ? k_pool + base + (long long)(head - nh) * head_stride : nullptr;
        if (ch < pair_chunks) {
            const int i = ch * VN;
            uint4 a = *reinterpret_cast<const uint4*>(h + i), b = *reinterpret_cast<const uint4*>(h + i + half), oa, ob;
            if (cs && !have_angles) load_angles(i);
            have_angles = false;
            const T* ae = reinterpret_cast<const T*>(&a);
            const T* be = reinterpret_cast<const T*>(&b);
            T* oae = reinterpret_cast<T*>(&oa);
            T* obe = reinterpret_cast<T*>(&ob);
#pragma unroll
            for (int e = 0; e < VN; ++e) {
                const float x1 = to_float<T>(ae[e]), x2 = to_float<T>(be[e]);
                float y1 = x1, y2 = x2;
                if (cs) {
                    y1 = __fsub_rn(__fmul_rn(x1, c[e]), __fmul_rn(x2, sn[e]));     // every product rounded, as the reference does
                    y2 = __fadd_rn(__fmul_rn(x2, c[e]), __fmul_rn(x1, sn[e]));
                }
                oae[e] = from_float<T>(y1);
                obe[e] = from_float<T>(y2);
            }
            if (!is_k) {
                *reinterpret_cast<uint4*>(h + i) = oa;
                *reinterpret_cast<uint4*>(h + i + half) = ob;
            } else if (dst) {
                *reinterpret_cast<uint4*>(dst + i) = oa;
                *reinterpret_cast<uint4*>(dst + i + half) = ob;
            }
        } else if (is_k && dst) {
            const int d = rot + (ch - pair_chunks) * VN;
            *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(h + d);
        }
    }
    if (base >= 0) {
        const T* v = row + (long long)(nh + nkv) * hd;
        const int chunks_per_head = hd / VN;
        for (int w = threadIdx.x; w < nkv * chunks_per_head; w += blockDim.x) {
            const int head = w / chunks_per_head, d = (w % chunks_per_head) * VN;
            *reinterpret_cast<uint4*>(v_pool + base + (long long)head * head_stride + d) =
                *reinterpret_cast<const uint4*>(v + (long long)head * hd + d);
        }
    }
}

TS_API int ts_rope_store(void* qkv, const int* positions, const int* seq_of_token, const float* table, int table_rows,
                         int rot, const int* block_table, int table_width, void* k_pool, void* v_pool,
                         long long page_stride, long long entry_offset, int page_tokens, int num_pages,
                         int num_tokens, int nh, int nkv, int hd, int write_kv, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && nh > 0 && nkv > 0 && hd > 0, "rope_store: bad sizes");
    TS_REQUIRE(hd % 2 == 0, "rope_store: head_dim %d must be even", hd);
    if (table) TS_REQUIRE(rot > 0 && rot % 2 == 0 && rot <= hd, "rope_store: rotary width %d does not fit head_dim %d", rot, hd);
    else rot = 0;
    TS_REQUIRE(page_tokens > 0 && table_width > 0, "rope_store: bad page geometry");
    (void)table_rows;
    if (num_tokens == 0) return 0;
    KVGeometry geo{page_stride, entry_offset, page_tokens, num_pages};
    const int threads = 256;
    const int vn = dtype == TS_F32 ? 4 : 8;
    const bool aligned = (uintptr_t)qkv % 16 == 0 && (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0 &&
                         page_stride % vn == 0 && entry_offset % vn == 0 && (uintptr_t)table % 16 == 0;
    if ((dtype == TS_F32 || dtype == TS_BF16) && aligned && hd % vn == 0 && (rot / 2) % vn == 0) {
        const int work = (nh + nkv) * ((rot / 2 + hd - rot) / vn);
        const int vthreads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
        if (dtype == TS_F32)
            TS_CHAINED_CHECK("rope_store", launch_chained(rope_store_vec_kernel<float, 4>, dim3(num_tokens), dim3(vthreads),
                                                          0, stream, (float*)qkv, positions, seq_of_token, table, rot,
                                                          block_table, table_width, (float*)k_pool, (float*)v_pool, geo,
                                                          nh, nkv, hd, write_kv));
        else
            TS_CHAINED_CHECK("rope_store", launch_chained(rope_store_vec_kernel<__nv_bfloat16, 8>, dim3(num_tokens),
                                                          dim3(vthreads), 0, stream, (__nv_bfloat16*)qkv, positions,
                                                          seq_of_token, table, rot, block_table, table_width,
                                                          (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, geo, nh, nkv,
                                                          hd, write_kv));
        return 0;
    }
    if (dtype == TS_F32)
        rope_store_kernel<float><<<num_tokens, threads, 0, stream>>>((float*)qkv, positions, seq_of_token, table, rot,
                                                                    block_table, table_width, (float*)k_pool,
                                                                    (float*)v_pool, geo, nh, nkv, hd, write_kv);
    else if (dtype == TS_BF16)
        rope_store_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, positions, seq_of_token, table, rot, block_table, table_width,
            (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, geo, nh, nkv, hd, write_kv);
    else
        return ts_fail("rope_store: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("rope_store");
    return 0;
}
