// Paged causal grouped-query attention for bfloat16 on tensor cores (mma.sync m16n8k16, float32
// accumulation), for head sizes 64 and 128 and pages of a multiple of 64 tokens.  Other sizes go
// to the generic kernel.  Two kernels share one tile routine:
//
//  * prefill: a CTA takes 64 consecutive tokens of one request for one query head and walks the
//    request's keys in tiles of 64 through a two-stage cp.async pipeline, online softmax in float32.
//    It serves whole prompts and portions over a cached prefix: a query at position p sees keys
//    max(0, p - window + 1) .. p (attention/torch_paged.py:36-45 of the reference, by positions).
//  * decode: requests that feed one token.  The g query heads that share a kv head are the rows of
//    one tile; the keys are cut into splits of 256 (fixed by key index, so the sums do not depend on
//    the batch); a CTA takes one split, each of its warps one tile of 64 keys; warps merge in
//    shared memory and write (max, sum, output) partials to scratch; a second kernel combines the
//    splits of each head.  The kernel is bound by the length of a warp's instruction stream, not by
//    the tensor pipe or by memory: tiles are loaded with folded addresses, tiles that are wholly
//    visible skip the mask, the padding rows of the tile skip the softmax, the fresh state skips the
//    rescale, and what does not depend on the kernel ahead on the stream is read before the wait
//    for it.
//
// Keys and values beyond the request's length (the unwritten tail of its last page) are zero-filled
// on load and masked by select, so whatever those slots hold never reaches a result.
#include "attention_bf16.h"

#include "common.cuh"

namespace {

constexpr int TILE = 64;           // keys per tile, queries per prefill CTA
constexpr int DW = 4;              // warps of a decode CTA, one tile of DKT keys each
constexpr int DKT = 64;            // keys per warp of a decode CTA
constexpr int SPLIT = DW * DKT;     // keys per decode split
static_assert(DKT % 16 == 0 && TILE % DKT == 0, "a decode tile is a multiple of 16 keys and divides a prefill tile (and so a page)");
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;                       // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x for x <= 0 (and -inf): one instruction; results below the normal range flush to zero.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile in shared memory: ROWS rows of HD bfloat16, 16-byte chunks XOR-swizzled by the row.
template <int HD>
__device__ __forceinline__ __nv_bfloat16* tile_at(__nv_bfloat16* tile, int row, int chunk) {
    return tile + row * HD + ((chunk ^ (row & 7)) << 3);
}

// Loads `rows` rows of HD bfloat16 (row r from src + r * src_stride) into a swizzled tile with the
// `nthreads` threads given; rows >= valid_rows are zero-filled.
template <int HD>
__device__ __forceinline__ void load_tile(__nv_bfloat16* tile, const __nv_bfloat16* src, long long src_stride,
                                          int rows, int valid_rows, int tid, int nthreads) {
    constexpr int CHUNKS = HD / 8;
    for (int i = tid; i < rows * CHUNKS; i += nthreads) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const bool ok = r < valid_rows;
        cp_async16(tile_at<HD>(tile, r, c), src + (ok ? (long long)r * src_stride + c * 8 : 0), ok);
    }
}

// One warp loads a tile whose ROWS rows lie back to back in memory (a head's keys of one page).
// Lane l takes 16-byte chunk l % CHUNKS of rows l / CHUNKS + j * (32 / CHUNKS): the row is
// r0 | const_j, so its swizzle is (chunk ^ r0) ^ const_j and every address is one base plus constants.
template <int HD, int ROWS, bool FULL>
__device__ __forceinline__ void load_tile_warp(__nv_bfloat16* tile, const __nv_bfloat16* src, int valid_rows, int lane) {
    constexpr int CHUNKS = HD / 8, RPI = 32 / CHUNKS;      // rows per iteration: 4 (head 64) or 2 (head 128)
    static_assert(ROWS % RPI == 0 && RPI <= 8, "tile rows must be a multiple of the rows one pass covers");
    const int c = lane % CHUNKS, r0 = lane / CHUNKS;
    const uint32_t base = smem_u32(tile) + r0 * HD * 2;
    const uint32_t swz = (uint32_t)(c ^ r0) << 4;
    const __nv_bfloat16* g = src + lane * 8;
#pragma unroll
    for (int j = 0; j < ROWS / RPI; ++j) {
        const uint32_t dst = base + j * RPI * HD * 2 + (swz ^ (((j * RPI) & 7) << 4));
        const int bytes = (FULL || r0 + j * RPI < valid_rows) ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(FULL || bytes ? g + j * RPI * HD : src), "r"(bytes));
    }
}

// Running softmax state of the two rows a thread owns (lane/4 and lane/4 + 8 of the warp's 16).
template <int HD>
struct RowState {
    float m[2] = {-INFINITY, -INFINITY};    // running maximum of score * scale * log2(e)
    float l[2] = {0.f, 0.f};                // this thread's share of the running sum
    float o[HD / 8][4];
    __device__ RowState() {
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    }
};

// One tile of KT keys against the warp's 16 query rows.  q: the rows' A fragments; k_tile/v_tile:
// swizzled [64][HD]; key0: index of the tile's first key; pos[2]: positions of the thread's two rows
// (keys lo[i]..pos[i] are visible).
// FIRST: the state is fresh (no key seen yet), so there is nothing to rescale.  TOP: only rows 0..7 of
// the tile are real (a decode group of at most 8 heads); the softmax of rows 8..15 is skipped, their
// probabilities are zero.
template <int HD, bool MASK, int KT = TILE, bool FIRST = false, bool TOP = false>
__device__ __forceinline__ void attend_tile(RowState<HD>& st, const uint32_t (&q)[HD / 16][4], __nv_bfloat16* k_tile,
                                            __nv_bfloat16* v_tile, int key0, const int (&pos)[2], const int (&lo)[2],
                                            float scale_log2, int lane) {
    float s[KT / 8][4];
#pragma unroll
    for (int n = 0; n < KT / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
    // S = Q K^T
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int nb = 0; nb < KT / 16; ++nb) {
            uint32_t b[4];
            const int row = nb * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int chunk = kk * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b, tile_at<HD>(k_tile, row, chunk));
            mma_bf16(s[2 * nb], q[kk], b[0], b[1]);
            mma_bf16(s[2 * nb + 1], q[kk], b[2], b[3]);
        }
    }
    // mask, running maximum (of raw scores; the scale is positive and joins the exponent below)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
        for (int e = 0; e < (TOP ? 2 : 4); ++e) {
            const int r = e >> 1;
            if (MASK) {                                   // tiles wholly inside every row's range skip the test
                const int key = key0 + n * 8 + ((lane & 3) << 1) + (e & 1);
                if (!(key <= pos[r] && key >= lo[r])) s[n][e] = -INFINITY;
            }
            tile_max[r] = fmaxf(tile_max[r], s[n][e]);
        }
    }
    float corr[2] = {1.f, 1.f}, m_use[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < (TOP ? 1 : 2); ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float m_new = fmaxf(st.m[r], tile_max[r] * scale_log2);   // -inf stays -inf
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;          // a row that has seen no key yet
        corr[r] = fast_exp2(st.m[r] - m_use[r]);              // 0 when the old maximum was -inf
        st.m[r] = m_new;
        st.l[r] *= corr[r];
    }
    if (!FIRST) {
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            st.o[n][0] *= corr[0]; st.o[n][1] *= corr[0];
            st.o[n][2] *= corr[1]; st.o[n][3] *= corr[1];
        }
    }
    // P = exp2(S - m), sums in float32, P rounded to bfloat16 for the second product
    uint32_t p[KT / 16][4];
#pragma unroll
    for (int n = 0; n < KT / 8; ++n) {
        const float p0 = fast_exp2(fmaf(s[n][0], scale_log2, -m_use[0])), p1 = fast_exp2(fmaf(s[n][1], scale_log2, -m_use[0]));
        float p2 = 0.f, p3 = 0.f;
        if (!TOP) {
            p2 = fast_exp2(fmaf(s[n][2], scale_log2, -m_use[1]));
            p3 = fast_exp2(fmaf(s[n][3], scale_log2, -m_use[1]));
        }
        st.l[0] += p0 + p1;
        st.l[1] += p2 + p3;
        p[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
        p[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
        for (int nb = 0; nb < HD / 16; ++nb) {
            uint32_t b[4];
            const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int chunk = nb * 2 + (lane >> 4);
            ldmatrix_x4_trans(b, tile_at<HD>(v_tile, row, chunk));
            mma_bf16(st.o[2 * nb], p[kk], b[0], b[1]);
            mma_bf16(st.o[2 * nb + 1], p[kk], b[2], b[3]);
        }
    }
}

struct AttnParams {
    const __nv_bfloat16* qkv;
    __nv_bfloat16* out;
    const __nv_bfloat16* k_pool;
    const __nv_bfloat16* v_pool;
    KVGeometry geo;
    const int* block_table;
    int table_width;
    const int* cu_q;
    const int* ctx_lens;
    int num_seqs, nh, nkv;
    float scale_log2;
    int window;
    const int* prefill_seqs;   // requests that feed more than one token, for the prefill grid (-1: none); null: every request
    // decode only
    float* partial_o;      // [seq][head][split][HD]
    float* partial_ml;     // [seq][head][split][2]
    int max_splits;
};

// Address of key (or value) row `key` of kv head `kvh` of the request whose table is given; null if
// the page was given back.
template <int HD>
__device__ __forceinline__ const __nv_bfloat16* kv_row_of_page(const __nv_bfloat16* pool, const KVGeometry& geo, int page,
                                                               int kvh, int key) {
    if (page < 0 || page >= geo.num_pages) return nullptr;
    return pool + (long long)page * geo.page_stride + geo.entry_offset + ((long long)kvh * geo.page_tokens + key % geo.page_tokens) * HD;
}
template <int HD>
__device__ __forceinline__ const __nv_bfloat16* kv_row(const __nv_bfloat16* pool, const KVGeometry& geo,
                                                       const int* table, int kvh, int key) {
    return kv_row_of_page<HD>(pool, geo, table[key / geo.page_tokens], kvh, key);
}

// ------------------------------------------------------------------------------------------------ prefill
template <int HD>
__global__ void __launch_bounds__(128) prefill_attention_kernel(AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);             // [64][HD]
    __nv_bfloat16* kv_tiles = q_tile + TILE * HD;                                     // 2 stages x (K, V) x [64][HD]
    const int seq = p.prefill_seqs ? p.prefill_seqs[blockIdx.z] : (int)blockIdx.z, head = blockIdx.y;
    if (seq < 0) return;                                                              // a padding entry of the list (a step replayed from a graph)
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    if (q_len <= 1) return;                                                           // decode rows go to the other kernel
    const int tiles = (q_len + TILE - 1) / TILE;
    const int tile_index = tiles - 1 - (int)blockIdx.x;                               // long tiles first
    if (tile_index < 0) return;
    const int ctx = p.ctx_lens[seq];
    const int row0 = tile_index * TILE;                                               // first query of the tile, within the step
    const int rows = min(TILE, q_len - row0);
    const int pos0 = ctx - q_len + row0;                                              // position of that query
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = head / (p.nh / p.nkv);
    const int row_width = (p.nh + 2 * p.nkv) * HD;
    const int* table = p.block_table + (long long)seq * p.table_width;

    load_tile<HD>(q_tile, p.qkv + (long long)(q_begin + row0) * row_width + (long long)head * HD, row_width, TILE, rows,
                  tid, 128);
    cp_async_commit();

    const int last_pos = pos0 + rows - 1;
    const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int kt_begin = first_key / TILE, kt_end = last_pos / TILE + 1;

    auto issue = [&](int kt, int stage) {
        __nv_bfloat16* k_tile = kv_tiles + stage * 2 * TILE * HD;
        __nv_bfloat16* v_tile = k_tile + TILE * HD;
        const int key0 = kt * TILE;
        const __nv_bfloat16* k_src = kv_row<HD>(p.k_pool, p.geo, table, kvh, key0);
        const __nv_bfloat16* v_src = kv_row<HD>(p.v_pool, p.geo, table, kvh, key0);
        const int valid = k_src ? min(TILE, ctx - key0) : 0;
        load_tile<HD>(k_tile, k_src ? k_src : p.k_pool, HD, TILE, valid, tid, 128);
        load_tile<HD>(v_tile, v_src ? v_src : p.v_pool, HD, TILE, valid, tid, 128);
        cp_async_commit();
    };

    cp_async_wait<0>();                      // the query tile has landed
    __syncthreads();
    issue(kt_begin, 0);
    uint32_t q[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(q[kk], tile_at<HD>(q_tile, row, kk * 2 + (lane >> 4)));
    }
    int pos[2], lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int tile_row = warp * 16 + (lane >> 2) + r * 8;
        pos[r] = tile_row < rows ? pos0 + tile_row : -1;                              // -1: a padding row sees nothing
        lo[r] = p.window > 0 ? max(0, pos[r] - p.window + 1) : 0;
    }
    RowState<HD> st;
    // positions of the warp's first and last real row: tiles wholly visible to all 16 rows need no mask
    const int warp_rows = min(rows - warp * 16, 16);
    const int warp_first = pos0 + warp * 16, warp_last = warp_first + warp_rows - 1;
    const int warp_lo_last = p.window > 0 ? max(0, warp_last - p.window + 1) : 0;
    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int stage = (kt - kt_begin) & 1;
        cp_async_wait<0>();                  // tile kt has landed (this thread's share)
        __syncthreads();                     // ... everyone's; and everyone is done with the other stage
        if (kt + 1 < kt_end) issue(kt + 1, stage ^ 1);
        __nv_bfloat16* k_tile = kv_tiles + stage * 2 * TILE * HD;
        const int key0 = kt * TILE;
        if (warp_rows > 0 && key0 <= warp_last) {           // else: all of the warp's rows lie before this tile
            if (warp_rows == 16 && key0 + TILE - 1 <= warp_first && key0 >= warp_lo_last)
                attend_tile<HD, false>(st, q, k_tile, k_tile + TILE * HD, key0, pos, lo, p.scale_log2, lane);
            else
                attend_tile<HD, true>(st, q, k_tile, k_tile + TILE * HD, key0, pos, lo, p.scale_log2, lane);
        }
    }
    // rows' sums over the quad, then write
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int tile_row = warp * 16 + (lane >> 2) + r * 8;
        if (tile_row >= rows) continue;
        const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
        __nv_bfloat16* o = p.out + ((long long)(q_begin + row0 + tile_row) * p.nh + head) * HD + ((lane & 3) << 1);
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(o + n * 8) =
                __floats2bfloat162_rn(st.o[n][2 * r] * inv, st.o[n][2 * r + 1] * inv);
    }
}

// ------------------------------------------------------------------------------------------------ decode
template <int HD>
__global__ void __launch_bounds__(DW * 32) decode_attention_kernel(AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    // Before the wait for the kernel ahead on the stream: what does not depend on it.  The index
    // data was written by the host before the step, and the keys and values of earlier steps lie
    // in the pages already; the kernel ahead (rotary + store) writes this step's query and the
    // one new key and value, so only the tile that holds position ctx - 1 is read after the wait.
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the page of this warp's keys is asked for together with the request's lengths, not after them: which
    // entry of the table it is follows from the grid alone (the entry is -1, or unused, where the request is shorter)
    const int key0 = split * SPLIT + warp * DKT;
    const int page0 = p.block_table[(long long)seq * p.table_width + min(key0 / p.geo.page_tokens, p.table_width - 1)];
    const int q_begin = p.cu_q[seq];
    const bool decoding = p.cu_q[seq + 1] - q_begin == 1;
    const int ctx = p.ctx_lens[seq];
    const int pos = ctx - 1;
    const int g = p.nh / p.nkv;
    const int first_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int key_begin = split * SPLIT;
    const bool active = decoding && key_begin <= pos && key_begin + SPLIT > first_key;
    float* part_o = p.partial_o + (((long long)seq * p.nh + kvh * g) * p.max_splits + split) * HD;
    float* part_ml = p.partial_ml + (((long long)seq * p.nh + kvh * g) * p.max_splits + split) * 2;
    if (!active) {
        chain_wait();
        chain_release();
        if (decoding && split < p.max_splits && tid < g) {     // an empty split: the combine skips it
            part_ml[(long long)tid * p.max_splits * 2] = -INFINITY;
            part_ml[(long long)tid * p.max_splits * 2 + 1] = 0.f;
        }
        return;
    }
    // shared memory: one query tile [16][HD], then per warp a key tile and a value tile [DKT][HD]
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* k_tile = q_tile + 16 * HD + warp * 2 * DKT * HD;
    __nv_bfloat16* v_tile = k_tile + DKT * HD;
    const int row_width = (p.nh + 2 * p.nkv) * HD;
    const bool warp_active = key0 <= pos && key0 + DKT > first_key;
    const bool holds_new = warp_active && key0 + DKT > pos;
    const __nv_bfloat16 *k_src = nullptr, *v_src = nullptr;
    int valid = 0;
    if (warp_active) {
        k_src = kv_row_of_page<HD>(p.k_pool, p.geo, page0, kvh, key0);
        v_src = kv_row_of_page<HD>(p.v_pool, p.geo, page0, kvh, key0);
        valid = k_src ? min(DKT, ctx - key0) : 0;
        if (!holds_new) {
            if (k_src) {
                load_tile_warp<HD, DKT, true>(k_tile, k_src, DKT, lane);
                load_tile_warp<HD, DKT, true>(v_tile, v_src, DKT, lane);
            } else {                                           // the page was given back: zeros
                load_tile_warp<HD, DKT, false>(k_tile, p.k_pool, 0, lane);
                load_tile_warp<HD, DKT, false>(v_tile, p.v_pool, 0, lane);
            }
            cp_async_commit();
        }
    }
    chain_wait();
    chain_release();
    RowState<HD> st;
    // rows 0..g-1 of the query tile are the g heads of this kv head; the rest are zero
    load_tile<HD>(q_tile, p.qkv + (long long)q_begin * row_width + (long long)kvh * g * HD, HD, 16, g, tid, DW * 32);
    if (holds_new) {
        load_tile_warp<HD, DKT, false>(k_tile, k_src ? k_src : p.k_pool, valid, lane);
        load_tile_warp<HD, DKT, false>(v_tile, v_src ? v_src : p.v_pool, valid, lane);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();                                           // the query tile is every warp's
    if (warp_active) {
        uint32_t q[HD / 16][4];
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
            ldmatrix_x4(q[kk], tile_at<HD>(q_tile, row, kk * 2 + (lane >> 4)));
        }
        const int posv[2] = {pos, pos};
        const int lov[2] = {first_key, first_key};
        const bool masked = holds_new || key0 < first_key;     // else every key of the tile is visible
        if (g <= 8) {
            if (masked) attend_tile<HD, true, DKT, true, true>(st, q, k_tile, v_tile, key0, posv, lov, p.scale_log2, lane);
            else attend_tile<HD, false, DKT, true, true>(st, q, k_tile, v_tile, key0, posv, lov, p.scale_log2, lane);
        } else {
            if (masked) attend_tile<HD, true, DKT, true, false>(st, q, k_tile, v_tile, key0, posv, lov, p.scale_log2, lane);
            else attend_tile<HD, false, DKT, true, false>(st, q, k_tile, v_tile, key0, posv, lov, p.scale_log2, lane);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
        }
    }
    __syncthreads();                                           // tiles are done with: reuse the memory for the merge
    // Only the g real rows are merged.  A row of the merge buffer is HD + 8 floats long, so that the
    // 8-byte stores of a warp (rows lane / 4, dims 2 * (lane % 4) + 8 n) fall into different banks.
    constexpr int RS = HD + 8;
    float* merge_o = reinterpret_cast<float*>(smem_raw);       // [warps][16 rows][RS]
    float* merge_ml = merge_o + DW * 16 * RS;                   // [warps][16 rows][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + r * 8;
        if (row >= g) continue;
        float* o = merge_o + ((warp * 16 + row) * RS) + ((lane & 3) << 1);
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) *reinterpret_cast<float2*>(o + n * 8) = make_float2(st.o[n][2 * r], st.o[n][2 * r + 1]);
        if ((lane & 3) == 0) *reinterpret_cast<float2*>(merge_ml + (warp * 16 + row) * 2) = make_float2(st.m[r], st.l[r]);
    }
    __syncthreads();
    // rows 0..g-1: merge the warps in order, one thread per (row, dim)
    for (int i = tid; i < g * HD; i += DW * 32) {
        const int row = i / HD, d = i % HD;
        float2 ml[DW];
        float ov[DW];
#pragma unroll
        for (int w = 0; w < DW; ++w) {
            ml[w] = *reinterpret_cast<const float2*>(merge_ml + (w * 16 + row) * 2);
            ov[w] = merge_o[(w * 16 + row) * RS + d];
        }
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < DW; ++w) m = fmaxf(m, ml[w].x);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < DW; ++w) {
            const float f = ml[w].x == -INFINITY ? 0.f : fast_exp2(ml[w].x - m);
            l += ml[w].y * f;
            o += ov[w] * f;
        }
        part_o[(long long)row * p.max_splits * HD + d] = o;
        if (d == 0) {
            part_ml[(long long)row * p.max_splits * 2] = m;
            part_ml[(long long)row * p.max_splits * 2 + 1] = l;
        }
    }
}

// One block per (request, head): merges the splits and writes the output row.  The block is GROUPS groups
// of HD threads (one per dim); a group takes a contiguous share of the splits, loads a chunk of them at
// once (so that it pays a memory latency or two, not one per split) and merges them in order against its
// own maximum; the groups' results are merged in group order.  A request of up to one chunk of splits is
// merged by the first group alone, and longer ones are always shared among 256 / HD groups (the launch
// has them whenever the step's longest request needs them): how a request's splits are merged depends on
// its own length only, never on what else is in the step.
constexpr int COMBINE_CHUNK = 16;
template <int HD, int GROUPS>
__global__ void __launch_bounds__(GROUPS * HD) decode_combine_kernel(AttnParams p) {
    __shared__ float group_o[GROUPS][HD];
    __shared__ float2 group_ml[GROUPS];
    const int seq = blockIdx.y, head = blockIdx.x;
    const int q_begin = p.cu_q[seq];              // index data: written by the host before the step
    const int q_len = p.cu_q[seq + 1] - q_begin;
    const int ctx = p.ctx_lens[seq];
    chain_wait();
    chain_release();
    if (q_len != 1) return;
    const int splits = (ctx + SPLIT - 1) / SPLIT;
    const float* part_o = p.partial_o + ((long long)seq * p.nh + head) * p.max_splits * HD;
    const float2* part_ml = reinterpret_cast<const float2*>(p.partial_ml) + ((long long)seq * p.nh + head) * p.max_splits;
    const int group = threadIdx.x / HD, d = threadIdx.x % HD;
    const int share = splits <= COMBINE_CHUNK ? splits : (splits + GROUPS - 1) / GROUPS;
    const int s_begin = min(group * share, splits), s_end = min(s_begin + share, splits);
    constexpr int CH = COMBINE_CHUNK;
    float2 ml[CH];
    float ov[CH];
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const bool ok = s_begin + j < s_end;
        ml[j] = ok ? part_ml[s_begin + j] : make_float2(-INFINITY, 0.f);
        ov[j] = ok ? part_o[(long long)(s_begin + j) * HD + d] : 0.f;
    }
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < CH; ++j) m = fmaxf(m, ml[j].x);
    for (int s = s_begin + CH; s < s_end; ++s) m = fmaxf(m, part_ml[s].x);
    float l = 0.f, o = 0.f;
    for (int s0 = s_begin; s0 < s_end; s0 += CH) {
        if (s0 > s_begin) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                const bool ok = s0 + j < s_end;
                ml[j] = ok ? part_ml[s0 + j] : make_float2(-INFINITY, 0.f);
                ov[j] = ok ? part_o[(long long)(s0 + j) * HD + d] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            if (ml[j].x == -INFINITY) continue;           // an empty split (its partial output was never written)
            const float f = fast_exp2(ml[j].x - m);
            l += ml[j].y * f;
            o += ov[j] * f;
        }
    }
    group_o[group][d] = o;
    if (d == 0) group_ml[group] = make_float2(m, l);
    __syncthreads();
    if (group != 0) return;
    float top = -INFINITY;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) top = fmaxf(top, group_ml[g].x);
    l = 0.f, o = 0.f;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
        if (group_ml[g].x == -INFINITY) continue;         // a group without a key
        const float f = fast_exp2(group_ml[g].x - top);
        l += group_ml[g].y * f;
        o += group_o[g][d] * f;
    }
    p.out[((long long)q_begin * p.nh + head) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
}

template <int HD>
int launch(const AttnParams& p, int max_q_len, int min_q_len, int max_ctx_len, int num_prefill_seqs, cudaStream_t stream) {
    if (max_q_len > 1) {
        const size_t smem = (size_t)(TILE * HD + 4 * TILE * HD) * sizeof(__nv_bfloat16);
        auto kernel = prefill_attention_kernel<HD>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        dim3 grid((max_q_len + TILE - 1) / TILE, p.nh, p.prefill_seqs ? num_prefill_seqs : p.num_seqs);
        kernel<<<grid, 128, smem, stream>>>(p);
        TS_LAUNCH_CHECK("prefill_attention");
    }
    if (min_q_len <= 1) {
        const size_t tiles = (size_t)(16 + DW * 2 * DKT) * HD * sizeof(__nv_bfloat16);
        const size_t merge = (size_t)(DW * 16 * (HD + 8) + DW * 16 * 2) * sizeof(float);
        const size_t smem = tiles > merge ? tiles : merge;
        auto kernel = decode_attention_kernel<HD>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        const int splits = (max_ctx_len + SPLIT - 1) / SPLIT;
        if (splits > p.max_splits) return ts_fail("decode_attention: %d splits needed, scratch holds %d", splits, p.max_splits);
        dim3 grid(splits, p.nkv, p.num_seqs);
        TS_CHAINED_CHECK("decode_attention", launch_chained(kernel, grid, dim3(DW * 32), smem, stream, p));
        if (splits <= COMBINE_CHUNK)
            TS_CHAINED_CHECK("decode_combine", launch_chained(decode_combine_kernel<HD, 1>, dim3(p.nh, p.num_seqs), dim3(HD), 0,
                                                              stream, p));
        else
            TS_CHAINED_CHECK("decode_combine", launch_chained(decode_combine_kernel<HD, 256 / HD>, dim3(p.nh, p.num_seqs),
                                                              dim3(256), 0, stream, p));
    }
    return 0;
}

}  // namespace

// Scratch the decode path needs: floats for partial outputs and for (max, sum) pairs.
TS_API long long ts_attention_bf16_scratch_floats(int num_seqs, int nh, int hd, int max_ctx_len) {
    const long long splits = (max_ctx_len + SPLIT - 1) / SPLIT;
    return (long long)num_seqs * nh * splits * (hd + 2);
}

TS_API int ts_attention_bf16_supported(int hd, int page_tokens, int nh, int nkv) {
    return (hd == 64 || hd == 128) && page_tokens % TILE == 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= 16;
}

// The arguments are described in attention_bf16.h.  (A prefill CTA that only finds out it has nothing
// to do still holds its shared memory while it does: hence prefill_seqs.)
TS_API int ts_paged_attention_bf16(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                                   long long page_stride, long long entry_offset, int page_tokens, int num_pages,
                                   const int* block_table, int table_width, const int* cu_q, const int* ctx_lens,
                                   int num_seqs, int max_q_len, int min_q_len, int max_ctx_len, int nh, int nkv, int hd,
                                   float scale, int window, float* scratch, long long scratch_floats,
                                   const int* prefill_seqs, int num_prefill_seqs, cudaStream_t stream) {
    TS_REQUIRE(ts_attention_bf16_supported(hd, page_tokens, nh, nkv),
               "paged_attention_bf16: head_dim %d / page %d / heads %d:%d is not taken by the tensor-core kernels", hd,
               page_tokens, nh, nkv);
    TS_REQUIRE(num_seqs >= 0 && max_q_len >= min_q_len && window >= 0, "paged_attention_bf16: bad sizes");
    TS_REQUIRE(num_seqs <= 65535 && nh <= 65535, "paged_attention_bf16: more than 65535 requests or heads in a step");
    if (num_seqs == 0 || max_q_len <= 0) return 0;
    AttnParams p;
    p.qkv = (const __nv_bfloat16*)qkv;
    p.out = (__nv_bfloat16*)out;
    p.k_pool = (const __nv_bfloat16*)k_pool;
    p.v_pool = (const __nv_bfloat16*)v_pool;
    p.geo = KVGeometry{page_stride, entry_offset, page_tokens, num_pages};
    p.block_table = block_table;
    p.table_width = table_width;
    p.cu_q = cu_q;
    p.ctx_lens = ctx_lens;
    p.num_seqs = num_seqs;
    p.nh = nh;
    p.nkv = nkv;
    p.scale_log2 = scale * LOG2E;
    p.window = window;
    p.max_splits = (max_ctx_len + SPLIT - 1) / SPLIT;
    p.prefill_seqs = prefill_seqs;
    TS_REQUIRE(prefill_seqs == nullptr || (num_prefill_seqs >= 0 && num_prefill_seqs <= num_seqs),
               "paged_attention_bf16: %d prefill requests of %d", num_prefill_seqs, num_seqs);
    if (prefill_seqs != nullptr && num_prefill_seqs == 0) max_q_len = min_q_len < 1 ? min_q_len : 1;   // nothing for the prefill kernel
    p.partial_o = scratch;
    p.partial_ml = scratch ? scratch + (long long)num_seqs * nh * p.max_splits * hd : nullptr;
    if (min_q_len <= 1) {
        TS_REQUIRE(scratch != nullptr && scratch_floats >= ts_attention_bf16_scratch_floats(num_seqs, nh, hd, max_ctx_len),
                   "paged_attention_bf16: scratch of %lld floats is too small", scratch_floats);
        TS_REQUIRE((long long)table_width * page_tokens >= max_ctx_len,
                   "paged_attention_bf16: block tables of %d pages do not reach %d tokens", table_width, max_ctx_len);
    }
    if (hd == 64) return launch<64>(p, max_q_len, min_q_len, max_ctx_len, num_prefill_seqs, stream);
    return launch<128>(p, max_q_len, min_q_len, max_ctx_len, num_prefill_seqs, stream);
}
