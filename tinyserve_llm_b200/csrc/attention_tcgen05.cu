// Prefill attention on the fifth-generation tensor cores, head sizes 64 and 128, bfloat16, pages of a
// multiple of 64 tokens, no window.  A CTA takes 128 consecutive tokens of one request for one query head
// (head size 128: rows lie in shared memory as two sub-tiles of 64 dims, key tiles hold 64 keys, so that
// two CTAs still fit an SM's shared and tensor memory):
//
//   * S = Q K^T for a tile of 128 keys is one tcgen05.mma chain (A = the query tile, B = the key
//     tile, both brought into 128-byte-swizzled shared memory by TMA straight from the qkv matrix
//     and from the paged pool) into tensor memory;
//   * two threads of the eight softmax warps own query row r, which is lane r of tensor memory: each reads
//     its half of the row of S with tcgen05.ld into registers, they exchange their maxima, keep the
//     reference of the exponentials and the sum in float32, write P = exp2(S - m) as bfloat16 pairs into
//     tensor-memory columns of P's own (tcgen05.st) and rescale their halves of the row of O, which is
//     needed only when the maximum has grown by more than 2^8 since the reference was taken;
//   * O += P V is a second tcgen05.mma chain with A = P read from tensor memory and B = the value
//     tile as it lies in shared memory (dims contiguous: the MN-major operand form).
//
// Warp 8 is the TMA producer over a two-stage ring of key/value tiles, warp 9 allocates tensor memory
// and issues the MMAs, warps 0..7 are the softmax.  Hand-offs are mbarriers: kv_full (TMA bytes),
// s_done / stage_free / all_done (tcgen05.commit) and p_ready (256 thread arrivals).  When the softmax
// hands over P of a tile, the scores of the next tile are issued before this tile's O += P V, so that
// the next softmax begins under that product.  Two CTAs share an SM, so one's softmax runs under the
// other's MMAs.  A query at position p sees keys 0..p
// (attention/torch_paged.py:36-45 of the reference, by positions); value rows beyond the request's
// length are zeroed in shared memory before they are multiplied.
//
// Every mbarrier wait gives up after about two seconds and records where in an error word.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int QROWS = 128;                   // queries per CTA
constexpr int TMEM_COLS = 256;
// Sizes that follow from the head size.  A tile row of more than 64 dims lies in shared memory as
// sub-tiles of 64 dims (128 bytes, the widest row the 128-byte swizzle takes), one after the other.
template <int HD>
struct Shape {
    static constexpr int KEYS = HD == 64 ? 128 : 64;     // keys per tile: two CTAs must fit an SM
    static constexpr int SUBS = HD / 64;                           // sub-tiles of 64 dims
    static constexpr int SUB_Q = QROWS * 128, SUB_KV = KEYS * 128; // bytes of a sub-tile
    static constexpr int Q_BYTES = QROWS * HD * 2, KV_BYTES = KEYS * HD * 2, STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int O_COL = KEYS;       // S at columns 0..KEYS-1, O after it, P (bfloat16 pairs) after O
    static constexpr int P_COL = KEYS + HD;
    static_assert(HD == 64 || HD == 128, "head sizes 64 and 128");
    static_assert(P_COL + KEYS / 2 <= TMEM_COLS, "S, O and P must fit the allocation");
};
constexpr int SOFTMAX_WARPS = 8;             // two threads a query row: each takes half of the tile's keys and half of O's dims
constexpr int PRODUCER_WARP = SOFTMAX_WARPS, MMA_WARP = SOFTMAX_WARPS + 1, THREADS = (SOFTMAX_WARPS + 2) * 32;
constexpr long long WAIT_CYCLES = 4000000000ll;
constexpr uint32_t SUSPEND_NS = 1000000;      // a waiting thread may sleep this long in one try before it looks at the clock
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;          // in powers of two

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error, int code) {
    const long long start = clock64();
    uint32_t done = 0;
    while (true) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(smem_u32(bar)), "r"(parity), "r"(SUSPEND_NS) : "memory");
        if (done) return true;
        if (clock64() - start > WAIT_CYCLES) {
            atomicExch(error, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// 128-byte-swizzled tile of rows of 128 bytes; groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// bfloat16 x bfloat16 -> float32; A K-major (or in tensor memory); B K-major, or MN-major if b_mn.
__device__ __forceinline__ uint32_t instr_desc(int m, int n, bool b_mn) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= 1u << 7;
    d |= 1u << 10;
    if (b_mn) d |= 1u << 16;
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(m >> 4) << 24;
    return d;
}
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The two softmax warps of a quadrant meet at a named barrier of their own (ids 1..4; 0 is __syncthreads).
__device__ __forceinline__ void pair_barrier(int quadrant) {
    switch (quadrant) {
        case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
    }
}

struct FlashParams {
    __nv_bfloat16* out;               // [T, nh * HD]
    const int* block_table;
    int table_width;
    const int* cu_q;
    const int* ctx_lens;
    const int* prefill_seqs;          // requests that feed more than one token (-1: none); null: every request has CTAs
    int nh, nkv;
    int page_tokens, num_pages;
    int entries, entry;               // cache entries of the layer group; this layer's index among them
    float scale_log2;
    int* error;
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 2) prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                        const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v,
                                                                        FlashParams p) {
    using S_ = Shape<HD>;
    constexpr int KEYS = S_::KEYS, SUBS = S_::SUBS, SUB_Q = S_::SUB_Q, SUB_KV = S_::SUB_KV, Q_BYTES = S_::Q_BYTES,
                  KV_BYTES = S_::KV_BYTES, STAGE_BYTES = S_::STAGE_BYTES, O_COL = S_::O_COL, P_COL = S_::P_COL;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t q_full, kv_full[2], stage_free[2], s_done, p_ready, all_done;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    __shared__ float half_max[2][2][QROWS];          // [tile parity][half][row]: the two threads of a row exchange their maxima
    __shared__ float half_sum[2][QROWS];             // ... and, at the end, their sums

    // blockIdx.x (which varies fastest in the order CTAs are handed out) is the head, blockIdx.y counts the
    // request's tiles from its last: the tile with the most keys of every head starts first, and
    // the short ones fill the SMs as the long ones finish.
    const int seq = p.prefill_seqs ? p.prefill_seqs[blockIdx.z] : (int)blockIdx.z, head = blockIdx.x;
    chain_wait();                                    // q, k and v of the step come from kernels ahead on the stream
    if (seq < 0) return;                             // a padding entry of the list (a step replayed from a graph)
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    if (q_len <= 1) return;                          // decode rows go to the split-key kernels
    const int tiles = (q_len + QROWS - 1) / QROWS;
    const int tile_index = tiles - 1 - (int)blockIdx.y;
    if (tile_index < 0) return;
    const int ctx = p.ctx_lens[seq];
    const int row0 = tile_index * QROWS;
    const int rows = min(QROWS, q_len - row0);
    const int pos0 = ctx - q_len + row0;             // position of the tile's first query
    const int last_pos = pos0 + rows - 1;
    const int num_kv = last_pos / KEYS + 1;
    const int kvh = head / (p.nh / p.nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = p.block_table + (long long)seq * p.table_width;

    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = base;
    unsigned char* kv_tiles = base + Q_BYTES;        // stage s: K tile at s * STAGE_BYTES, V tile after it

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&stage_free[s], 1);
        }
        mbar_init(&s_done, 1);
        mbar_init(&p_ready, SOFTMAX_WARPS * 32);
        mbar_init(&all_done, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;
    // Dependents are let in only now that this CTA holds its tensor memory: a kernel behind this one that
    // allocates tensor memory before it waits for this grid could otherwise starve a CTA of this grid.
    chain_release();

    if (warp == PRODUCER_WARP && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
        for (int h = 0; h < SUBS; ++h) tma_load_2d(q_tile + h * SUB_Q, &map_q, &q_full, head * HD + h * 64, q_begin + row0);
        for (int j = 0; j < num_kv; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&stage_free[s], ((j >> 1) & 1) ^ 1, p.error, 11)) { failed = 1; break; }
            unsigned char* k_tile = kv_tiles + s * STAGE_BYTES;
            unsigned char* v_tile = k_tile + KV_BYTES;
            mbar_expect_tx(&kv_full[s], STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < KEYS / 64; ++b) {    // boxes of 64 keys x 64 dims: a box never crosses a page
                const int key = j * KEYS + b * 64;
                int page = table[min(key / p.page_tokens, p.table_width - 1)];
                if (page < 0 || page >= p.num_pages) page = 0;     // given back or beyond the request: masked anyway
                const int row = ((page * p.entries + p.entry) * p.nkv + kvh) * p.page_tokens + key % p.page_tokens;
#pragma unroll
                for (int h = 0; h < SUBS; ++h) {
                    tma_load_2d(k_tile + h * SUB_KV + b * (64 * 128), &map_k, &kv_full[s], h * 64, row);
                    tma_load_2d(v_tile + h * SUB_KV + b * (64 * 128), &map_v, &kv_full[s], h * 64, row);
                }
            }
        }
    } else if (warp == MMA_WARP && lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        const uint32_t idesc_s = instr_desc(QROWS, KEYS, false);
        const uint32_t idesc_o = instr_desc(QROWS, 64, true);        // O in column blocks of 64 dims, one per sub-tile of V
        bool ok = mbar_wait(&q_full, 0, p.error, 12);
        // S = Q K^T of tile j, once its keys have landed
        auto issue_scores = [&](int j) -> bool {
            const int s = j & 1;
            if (!mbar_wait(&kv_full[s], (j >> 1) & 1, p.error, 13)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < SUBS; ++h) {
                const uint64_t q_desc = smem_desc(q_tile + h * SUB_Q);
                const uint64_t k_desc = smem_desc(kv_tiles + s * STAGE_BYTES + h * SUB_KV);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_ss(tmem, q_desc + 2 * k, k_desc + 2 * k, idesc_s, (h | k) != 0);
            }
            umma_commit(&s_done);
            return true;
        };
        ok = ok && issue_scores(0);
        for (int j = 0; j < num_kv && ok; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&p_ready, j & 1, p.error, 14)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // The softmax has read S of tile j (P lies in columns of its own), so the next tile's scores go first:
            // its softmax can begin while O += P V of this tile is still running.  The softmax waits for that
            // product (stage_free) before it writes P again or rescales O.
            if (j + 1 < num_kv && !issue_scores(j + 1)) { ok = false; break; }
#pragma unroll
            for (int h = 0; h < SUBS; ++h) {         // O += P V: 16 keys are 8 columns of packed P and 16 rows (2048 bytes) of a V sub-tile
                const uint64_t v_desc = smem_desc(kv_tiles + s * STAGE_BYTES + KV_BYTES + h * SUB_KV);
#pragma unroll
                for (int k = 0; k < KEYS / 16; ++k)
                    umma_ts(tmem + O_COL + 64 * h, tmem + P_COL + 8 * k, v_desc + 128 * k, idesc_o, (j | k) != 0);
            }
            umma_commit(&stage_free[s]);
        }
        if (!ok) failed = 1;
        umma_commit(&all_done);
    } else if (warp < SOFTMAX_WARPS) {
        // ---------------------------------------------------------------- softmax: two threads own query row r
        // Warp w reads the tensor-memory lanes of quadrant w % 4 (a warp can reach no others); the two
        // warps of a quadrant split the tile's keys, and O's dims, in halves.  They exchange their
        // halves' maxima through shared memory once a tile, behind a barrier of their 64 threads.
        const int quadrant = warp & 3, half = warp >> 2;
        const int r = quadrant * 32 + lane;
        const int pos = r < rows ? pos0 + r : -1;    // -1: a padding row sees nothing
        const uint32_t lane_addr = tmem + ((uint32_t)(quadrant * 32) << 16);
        constexpr int HK = KEYS / 2, HO = HD / 2;    // this thread's keys of a tile, and its dims of O
        const int col0 = half * HK;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < num_kv; ++j) {
            const int s = j & 1;
            const int key0 = j * KEYS;
            // a wait that ran out: the warp (as one) skips the work of this and the later tiles but still meets its
            // partner at the barrier below and still arrives at p_ready, so that nobody is left waiting for it
            if (ok && !mbar_wait(&s_done, j & 1, p.error, 15)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                pair_barrier(quadrant);
                mbar_arrive(&p_ready);
                continue;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool masked = key0 + KEYS - 1 > pos0;        // some row of the tile does not see all of these keys
            // this thread's keys of S come into registers once, all loads under way together
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            uint32_t sv[HK / 32][32];
#pragma unroll
            for (int ch = 0; ch < HK / 32; ++ch) tmem_ld32(lane_addr + col0 + ch * 32, sv[ch]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // pass 1: the maximum over them (four running maxima: no long dependent chain)
#pragma unroll
            for (int ch = 0; ch < HK / 32; ++ch) {
                const int c = col0 + ch * 32;
                if (masked) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (key0 + c + i <= pos) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[ch][i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[ch][i]));
                }
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            half_max[j & 1][half][r] = mx;
            pair_barrier(quadrant);
            mx = fmaxf(mx, half_max[j & 1][half ^ 1][r]);
            // O += P V of the tile before must have retired before P is written again and O is rescaled
            if (j > 0 && !mbar_wait(&stage_free[(j - 1) & 1], ((j - 1) >> 1) & 1, p.error, 17)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                mbar_arrive(&p_ready);
                continue;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // The reference the exponentials are taken against follows the maximum only when that has grown by
            // more than RESCALE_STEP: until then P holds values up to 2^RESCALE_STEP, which float32 sums and
            // bfloat16 products take without loss, and O needs no rescaling (softmax does not depend on the
            // reference it is computed against).
            const float m_tile = mx * p.scale_log2;
            const bool moved = m_tile > m_run + RESCALE_STEP;          // also the first tile that shows the row a key
            const float m_new = moved ? m_tile : m_run;
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = moved ? fast_exp2(m_run - m_use) : 1.f;
            m_run = m_new;
            // pass 2: P = exp2(S * scale - m) as bfloat16 pairs into P's own columns (pair i covers keys 2i, 2i+1).
            // The tile on the diagonal has a loop of its own: inside one loop the compiler keeps the compare
            // and select of every element in the instruction stream of the tiles that need none.
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            if (masked) {
#pragma unroll
                for (int ch = 0; ch < HK / 32; ++ch) {
                    const int c = col0 + ch * 32;
                    uint32_t packed[16];
                    const uint32_t (&v)[32] = sv[ch];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use));
                        float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_use));
                        if (key0 + c + i > pos) p0 = 0.f;
                        if (key0 + c + i + 1 > pos) p1 = 0.f;
                        l4[(i >> 1) & 3] += p0 + p1;
                        packed[i >> 1] = pack_bf16(p0, p1);
                    }
                    tmem_st16(lane_addr + P_COL + (c >> 1), packed);
                }
            } else {
#pragma unroll
                for (int ch = 0; ch < HK / 32; ++ch) {
                    const int c = col0 + ch * 32;
                    uint32_t packed[16];
                    const uint32_t (&v)[32] = sv[ch];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_use));
                        l4[(i >> 1) & 3] += p0 + p1;
                        packed[i >> 1] = pack_bf16(p0, p1);
                    }
                    tmem_st16(lane_addr + P_COL + (c >> 1), packed);
                }
            }
            l_run = l_run * corr + ((l4[0] + l4[1]) + (l4[2] + l4[3]));
            // this thread's dims of O follow the new reference; skipped when no row of the warp moved it
            if (j > 0 && !__all_sync(0xffffffffu, corr == 1.f)) {
#pragma unroll 1
                for (int c = half * HO; c < half * HO + HO; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + O_COL + c, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                    tmem_st32(lane_addr + O_COL + c, v);
                }
            }
            // value rows beyond the request's length hold whatever the page held: zero them before they are multiplied
            if (half == 0 && r < KEYS && key0 + KEYS > ctx && key0 + r >= ctx) {
#pragma unroll
                for (int h = 0; h < SUBS; ++h) {
                    unsigned char* v_row = kv_tiles + s * STAGE_BYTES + KV_BYTES + h * SUB_KV + r * 128;
#pragma unroll
                    for (int i = 0; i < 128; i += 16) *reinterpret_cast<uint4*>(v_row + i) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&p_ready);
        }
        if (ok) ok = mbar_wait(&all_done, 0, p.error, 16);
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // the row's sum is the two halves' sums (both were kept against the same maxima)
        half_sum[half][r] = l_run;
        pair_barrier(quadrant);
        l_run += half_sum[half ^ 1][r];
        if (ok && !failed) {                         // every thread of the warp takes part in the loads; only real rows store
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* o = p.out + ((long long)(q_begin + row0 + r) * p.nh + head) * HD;
#pragma unroll 1
            for (int c = half * HO; c < half * HO + HO; c += 32) {
                uint32_t v[32];
                tmem_ld32(lane_addr + O_COL + c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r < rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 packed;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            h[e] = __floats2bfloat162_rn(__uint_as_float(v[i + 2 * e]) * inv, __uint_as_float(v[i + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(o + c + i) = packed;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(sym);
    }
    return fn;
}

// [rows, 64] bfloat16 view with a row stride of ld elements; boxes of box_rows x 64, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return ts_fail("attention_tcgen05: the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ts_fail("attention_tcgen05: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

}  // namespace

TS_API int ts_attention_tcgen05_supported(int hd, int page_tokens, int nh, int nkv, int window) {
    return (hd == 64 || hd == 128) && page_tokens % 64 == 0 && nkv > 0 && nh % nkv == 0 && window == 0;
}

// Prompt portions (requests that feed more than one token) of a step; requests that feed one token
// are left to the decode kernels.  prefill_seqs (optional, device) lists the former, so that the grid
// has no CTAs for the latter.  The pools are [pages][entries][kv heads][page_tokens][64].
TS_API int ts_prefill_attention_tcgen05(const void* qkv, void* out, const void* k_pool, const void* v_pool, int num_pages,
                                        int entries, int entry, int page_tokens, const int* block_table, int table_width,
                                        const int* cu_q, const int* ctx_lens, int num_seqs, int num_tokens, int max_q_len,
                                        int nh, int nkv, int hd, float scale, const int* prefill_seqs, int num_prefill_seqs,
                                        int* error, cudaStream_t stream) {
    TS_REQUIRE(ts_attention_tcgen05_supported(hd, page_tokens, nh, nkv, 0), "attention_tcgen05: sizes not taken (head_dim %d, page %d)", hd, page_tokens);
    TS_REQUIRE(error != nullptr, "attention_tcgen05: an error word is needed");
    TS_REQUIRE(num_seqs <= 65535 && (max_q_len + QROWS - 1) / QROWS <= 65535,
               "attention_tcgen05: more than 65535 requests, or tiles of a request, in a step");
    TS_REQUIRE(((uintptr_t)qkv % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0),
               "attention_tcgen05: operands must be 16-byte aligned");
    if (num_seqs == 0 || max_q_len <= 1) return 0;
    TS_REQUIRE(prefill_seqs == nullptr || (num_prefill_seqs >= 0 && num_prefill_seqs <= num_seqs),
               "attention_tcgen05: %d prefill requests of %d", num_prefill_seqs, num_seqs);
    if (prefill_seqs != nullptr && num_prefill_seqs == 0) return 0;
    const long long pool_rows = (long long)num_pages * entries * nkv * page_tokens;
    TS_REQUIRE(pool_rows < 0x7fffffffll, "attention_tcgen05: the pool has too many rows for 32-bit TMA coordinates");
    const long long row_width = (long long)(nh + 2 * nkv) * hd;
    CUtensorMap map_q, map_k, map_v;
    if (make_map(&map_q, qkv, num_tokens, row_width, row_width, QROWS)) return 1;
    if (make_map(&map_k, k_pool, pool_rows, hd, hd, 64)) return 1;
    if (make_map(&map_v, v_pool, pool_rows, hd, hd, 64)) return 1;
    FlashParams p;
    p.out = (__nv_bfloat16*)out;
    p.block_table = block_table;
    p.table_width = table_width;
    p.cu_q = cu_q;
    p.ctx_lens = ctx_lens;
    p.prefill_seqs = prefill_seqs;
    p.nh = nh;
    p.nkv = nkv;
    p.page_tokens = page_tokens;
    p.num_pages = num_pages;
    p.entries = entries;
    p.entry = entry;
    p.scale_log2 = scale * LOG2E;
    p.error = error;
    dim3 grid(nh, (max_q_len + QROWS - 1) / QROWS, prefill_seqs ? num_prefill_seqs : num_seqs);
    if (hd == 64) {
        const size_t smem = (size_t)Shape<64>::Q_BYTES + 2 * Shape<64>::STAGE_BYTES + 1024;
        auto kernel = prefill_attention_tcgen05_kernel<64>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TS_CHAINED_CHECK("attention_tcgen05", launch_chained(kernel, grid, dim3(THREADS), smem, stream, map_q, map_k, map_v, p));
    } else {
        const size_t smem = (size_t)Shape<128>::Q_BYTES + 2 * Shape<128>::STAGE_BYTES + 1024;
        auto kernel = prefill_attention_tcgen05_kernel<128>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TS_CHAINED_CHECK("attention_tcgen05", launch_chained(kernel, grid, dim3(THREADS), smem, stream, map_q, map_k, map_v, p));
    }
    return 0;
}
