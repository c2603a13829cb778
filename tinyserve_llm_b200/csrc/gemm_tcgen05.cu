// bfloat16 matrix product y = x . W^T on the fifth-generation tensor cores: operands staged in shared
// memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), tcgen05.mma issued by one thread, the
// float32 accumulator in tensor memory, read back with tcgen05.ld for the epilogue.
//
// Persistent: one CTA per SM walks over 128 x 256 tiles of y (two CTAs per SM over 128 x 128 tiles
// when there are few tiles), rows fastest, so that the CTAs running together share x in L2 while W streams.  Ten warps:
// warp 0 issues the TMA loads, warp 1 allocates tensor memory and issues the MMAs, warps 2..9 are
// the epilogue (each reads half the columns of the 32 accumulator lanes it may touch: with four warps the
// epilogue of a tile took longer than the tile's MMAs, and the tensor pipe waited for accumulators).  A ring of shared-memory stages
// is handed back and forth with mbarriers: `full` (TMA bytes landed) and `empty` (the MMAs that read
// the stage have retired, signalled by tcgen05.commit).  The accumulator is double-buffered in
// tensor memory (`tmem_full` / `tmem_empty`), so the epilogue of one tile runs under the main loop
// of the next.  Rows and columns beyond M, N and K are zero-filled by TMA and masked at the store.
//
// Epilogues: plain store (bfloat16 or float32), or SwiGLU: the tile's BN columns are BN/2 gate rows
// of W and the BN/2 up rows that belong to them, and it stores round(silu(gate)) * up
// (model/llama.py:80-83 of the reference), which saves writing and re-reading the [T, 2I] product.
//
// Every wait on an mbarrier gives up after about two seconds, records where in an error word the
// host can read, and the CTA goes on to free its tensor memory and return.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int EPI_WARPS = 8, THREADS = 64 + 32 * EPI_WARPS;     // two epilogue warps for each quarter of the accumulator's lanes
constexpr int A_BYTES = BM * BK * 2;
constexpr long long WAIT_CYCLES = 4000000000ll;     // about two seconds at 2 GHz

enum { EPI_STORE = 0, EPI_SWIGLU = 1 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// false: the wait ran out of time (the error word says which one)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error, int code) {
    const long long start = clock64();
    uint32_t done = 0;
    while (true) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
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

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16) with
// the 128-byte swizzle: start address, stride between groups of 8 rows (1024 bytes), sm_100 version.
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);          // bits 0..13: start address / 16
    d |= (uint64_t)1 << 16;                                      // bits 16..29: leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                            // bits 32..45: stride byte offset / 16
    d |= (uint64_t)1 << 46;                                      // bits 46..47: descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                      // bits 61..63: 128-byte swizzle
    return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, tile M x N.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
    uint32_t d = 0;
    d |= 1u << 4;                       // accumulator format: float32
    d |= 1u << 7;                       // A format: bfloat16
    d |= 1u << 10;                      // B format: bfloat16
    d |= (uint32_t)(n >> 3) << 17;      // N / 8
    d |= (uint32_t)(m >> 4) << 24;      // M / 16
    return d;
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {      // r: 32 registers (indices known at compile time)
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

struct GemmParams {
    void* y;
    int M, N, K;
    long long ldy;
    int inter;            // SwiGLU: rows of W per half
    int out_f32;
    int* error;
};

template <int EPI, int BN, int STAGES>
__global__ void __launch_bounds__(THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                           const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    constexpr int B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    // STAGES: 4 for wide tiles; 3 for narrow ones, of which two CTAs share an SM; 6 for narrow tiles when x has
    // a single tile of rows: then a CTA does one tile, nothing hides the latency of memory but the depth of
    // the ring, and the product is bound by the stream of W
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? BN / 2 : BN;          // output columns per tile
    constexpr int TMEM_COLS = 2 * BN;                                   // two accumulators
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.K + BK - 1) / BK;
    const int out_cols = EPI == EPI_SWIGLU ? p.inter : p.N;
    const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (out_cols + OUT_COLS - 1) / OUT_COLS;
    const int num_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full_bar[b], 1);
            mbar_init(&tmem_empty_bar[b], EPI_WARPS);   // one arrival per epilogue warp
        }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                 // one warp allocates the accumulators' columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    chain_wait();                                    // x may come from the kernel ahead on the stream
    chain_release();

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        int kg = 0;                                  // k-blocks issued so far, over all tiles
        for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * OUT_COLS;
            for (int kb = 0; kb < kblocks; ++kb, ++kg) {
                const int s = kg % STAGES;
                // a fresh barrier passes a wait on parity 1: the first round finds every stage free
                if (!mbar_wait(&empty_bar[s], ((kg / STAGES) & 1) ^ 1, p.error, 1)) { failed = 1; break; }
                unsigned char* a_tile = stages + s * STAGE_BYTES;
                unsigned char* b_tile = a_tile + A_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(a_tile, &map_a, &full_bar[s], kb * BK, m0);
                if (EPI == EPI_SWIGLU) {             // BN/2 gate rows, then the BN/2 up rows that go with them
                    tma_load_2d(b_tile, &map_b, &full_bar[s], kb * BK, n0);
                    tma_load_2d(b_tile + B_BYTES / 2, &map_b, &full_bar[s], kb * BK, p.inter + n0);
                } else {
                    tma_load_2d(b_tile, &map_b, &full_bar[s], kb * BK, n0);
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        const uint32_t idesc = instr_desc(BM, BN);
        int kg = 0, iter = 0;
        for (int tile = blockIdx.x; tile < num_tiles && !failed; tile += gridDim.x, ++iter) {
            const int buf = iter & 1;
            if (!mbar_wait(&tmem_empty_bar[buf], ((iter >> 1) & 1) ^ 1, p.error, 4)) { failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + buf * BN;
            for (int kb = 0; kb < kblocks; ++kb, ++kg) {
                const int s = kg % STAGES;
                if (!mbar_wait(&full_bar[s], (kg / STAGES) & 1, p.error, 2)) { failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t a_desc = smem_desc(stages + s * STAGE_BYTES);
                const uint64_t b_desc = smem_desc(stages + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)    // 16 elements of K are 32 bytes: the start address moves by 2 units of 16
                    umma(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                umma_commit(&empty_bar[s]);              // the stage is free once these MMAs have read it
            }
            umma_commit(&tmem_full_bar[buf]);            // the accumulator is complete once everything issued has retired
        }
    } else if (warp >= 2) {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;                // the 32 lanes of tensor memory this warp may read
        const int side = (warp - 2) >> 2;            // which half of the tile's columns: two warps share a quarter
        int iter = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++iter) {
            const int buf = iter & 1;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * OUT_COLS;
            if (!mbar_wait(&tmem_full_bar[buf], (iter >> 1) & 1, p.error, 3) || failed) { failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const uint32_t lane_addr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
            if (EPI == EPI_SWIGLU) {
                __nv_bfloat16* out = (__nv_bfloat16*)p.y + (long long)row * p.ldy + n0;
                // the warp's whole share of the accumulator into registers at once, so that the accumulator goes back
                // to the MMAs before the arithmetic and the stores, not after them
                constexpr int SHARE = BN / 4;
                const int c0 = side * SHARE;
                uint32_t gate[SHARE], up[SHARE];
#pragma unroll
                for (int cc = 0; cc < SHARE; cc += 32) {
                    tmem_ld32(lane_addr + c0 + cc, gate + cc);
                    tmem_ld32(lane_addr + BN / 2 + c0 + cc, up + cc);
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tmem_empty_bar[buf])) : "memory");
                if (row < p.M) {
#pragma unroll
                    for (int j = 0; j < SHARE; j += 8) {
                        const int c = c0 + j;
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float g = round_to<__nv_bfloat16>(__uint_as_float(gate[j + e]));
                            const float u = round_to<__nv_bfloat16>(__uint_as_float(up[j + e]));
                            v[e] = round_to<__nv_bfloat16>(__fdividef(g, 1.f + __expf(-g))) * u;
                        }
                        if (n0 + c + 8 <= p.inter && (((uintptr_t)(out + c)) & 15) == 0) {
                            uint4 packed;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                            for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                            *reinterpret_cast<uint4*>(out + c) = packed;
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (n0 + c + e < p.inter) out[c + e] = __float2bfloat16_rn(v[e]);
                        }
                    }
                }
            } else {
                constexpr int SHARE = BN / 2;
                const int c0 = side * SHARE;
                uint32_t acc[SHARE];
#pragma unroll
                for (int cc = 0; cc < SHARE; cc += 32) tmem_ld32(lane_addr + c0 + cc, acc + cc);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tmem_empty_bar[buf])) : "memory");
                if (row < p.M) {
#pragma unroll
                    for (int j = 0; j < SHARE; j += 8) {
                        const int c = c0 + j;
                        if (p.out_f32) {
                            float* out = (float*)p.y + (long long)row * p.ldy + n0 + c;
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (n0 + c + e < p.N) out[e] = __uint_as_float(acc[j + e]);
                        } else {
                            __nv_bfloat16* out = (__nv_bfloat16*)p.y + (long long)row * p.ldy + n0 + c;
                            if (n0 + c + 8 <= p.N && (((uintptr_t)out) & 15) == 0) {
                                uint4 v;
                                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    h[e] = __floats2bfloat162_rn(__uint_as_float(acc[j + 2 * e]), __uint_as_float(acc[j + 2 * e + 1]));
                                *reinterpret_cast<uint4*>(out) = v;
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    if (n0 + c + e < p.N) out[e] = __float2bfloat16_rn(__uint_as_float(acc[j + e]));
                            }
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// The same product with two CTAs on one tile (tcgen05 cta_group::2): a pair of CTAs on neighbouring SMs
// computes a 256 x 256 tile of y.  Each CTA loads its own 128 rows of x and HALF of the tile's rows of W
// (with SwiGLU: one the gate rows, the other the up rows), and the MMAs, issued by the pair's first CTA
// for both, read the halves of W out of both CTAs' shared memory.  Per SM and k-step that is 32 KB
// written by TMA and read by the tensor core instead of 48 KB, and shared memory's bandwidth is what
// bounds the single-CTA kernel.  Each CTA keeps the accumulator of its own 128 rows in its own tensor
// memory and runs its own epilogue.
//
// Who signals whom.  `full` lives in the first CTA: it expects the bytes of both CTAs' loads, and both
// CTAs' TMA loads count on it.  `empty` and `tmem_full` exist in both CTAs and are signalled in both at
// once by the first CTA's tcgen05.commit (multicast).  `tmem_empty` lives in the first CTA and counts
// the epilogue warps of both.  A cluster barrier after the barriers' initialisation keeps either CTA
// from signalling a barrier that does not exist yet, another before the tensor memory is given back
// keeps either from leaving while the other still reads its shared memory.
__device__ __forceinline__ uint32_t pair_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t in_first_cta(const void* local) {      // the same object in the pair's first CTA
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(0));
    return remote;
}
__device__ __forceinline__ void pair_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, uint32_t bar_in_first, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem)), "l"(map), "r"(bar_in_first), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {          // arrives on `bar` in both CTAs
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_in_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_in_cluster) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(THREADS) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    constexpr int BN = 256, STAGES = 6;
    constexpr int B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;      // per CTA: its rows of x, half of W's
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? BN / 2 : BN;
    constexpr int TMEM_COLS = 2 * BN;                                                 // two accumulators
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)pair_rank();
    const int kblocks = (p.K + BK - 1) / BK;
    const int out_cols = EPI == EPI_SWIGLU ? p.inter : p.N;
    const int m_tiles = (p.M + 2 * BM - 1) / (2 * BM), n_tiles = (out_cols + OUT_COLS - 1) / OUT_COLS;
    const int num_tiles = m_tiles * n_tiles;
    const int pair = blockIdx.x / 2, pairs = gridDim.x / 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full_bar[b], 1);
            mbar_init(&tmem_empty_bar[b], 2 * EPI_WARPS);   // one arrival per epilogue warp of both CTAs
        }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                 // one warp of each CTA allocates the pair's accumulators
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    pair_sync();                                     // both CTAs' barriers exist

    chain_wait();                                    // x may come from the kernel ahead on the stream
    chain_release();

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer (one in each CTA)
        int kg = 0;
        for (int tile = pair; tile < num_tiles && !failed; tile += pairs) {
            const int m0 = (tile % m_tiles) * 2 * BM + rank * BM, n0 = (tile / m_tiles) * OUT_COLS;
            // this CTA's half of the tile's rows of W
            const int w0 = EPI == EPI_SWIGLU ? (rank == 0 ? n0 : p.inter + n0) : n0 + rank * (BN / 2);
            for (int kb = 0; kb < kblocks; ++kb, ++kg) {
                const int s = kg % STAGES;
                if (!mbar_wait(&empty_bar[s], ((kg / STAGES) & 1) ^ 1, p.error, 1)) { failed = 1; break; }
                unsigned char* a_tile = stages + s * STAGE_BYTES;
                const uint32_t full = in_first_cta(&full_bar[s]);
                if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
                tma_load_2d_pair(a_tile, &map_a, full, kb * BK, m0);
                tma_load_2d_pair(a_tile + A_BYTES, &map_b, full, kb * BK, w0);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------------------------------------------------------- MMA issuer (the pair's first CTA only)
        const uint32_t idesc = instr_desc(2 * BM, BN);
        int kg = 0, iter = 0;
        for (int tile = pair; tile < num_tiles && !failed; tile += pairs, ++iter) {
            const int buf = iter & 1;
            if (!mbar_wait(&tmem_empty_bar[buf], ((iter >> 1) & 1) ^ 1, p.error, 4)) { failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + buf * BN;
            for (int kb = 0; kb < kblocks; ++kb, ++kg) {
                const int s = kg % STAGES;
                if (!mbar_wait(&full_bar[s], (kg / STAGES) & 1, p.error, 2)) { failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t a_desc = smem_desc(stages + s * STAGE_BYTES);
                const uint64_t b_desc = smem_desc(stages + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_pair(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                umma_commit_pair(&empty_bar[s]);         // the stage is free in both CTAs once these MMAs have read it
            }
            umma_commit_pair(&tmem_full_bar[buf]);       // both CTAs' halves of the accumulator are complete
        }
    } else if (warp >= 2) {
        // ---------------------------------------------------------------- epilogue (in each CTA, for its own rows)
        const int quarter = warp & 3;
        const int side = (warp - 2) >> 2;            // which half of the tile's columns: two warps share a quarter
        int iter = 0;
        for (int tile = pair; tile < num_tiles; tile += pairs, ++iter) {
            const int buf = iter & 1;
            const int m0 = (tile % m_tiles) * 2 * BM + rank * BM, n0 = (tile / m_tiles) * OUT_COLS;
            if (!mbar_wait(&tmem_full_bar[buf], (iter >> 1) & 1, p.error, 3) || failed) { failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const uint32_t lane_addr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
            const uint32_t drained = in_first_cta(&tmem_empty_bar[buf]);
            if (EPI == EPI_SWIGLU) {
                __nv_bfloat16* out = (__nv_bfloat16*)p.y + (long long)row * p.ldy + n0;
                // the warp's whole share of the accumulator into registers at once, so that the accumulator goes back
                // to the MMAs before the arithmetic and the stores, not after them
                constexpr int SHARE = BN / 4;
                const int c0 = side * SHARE;
                uint32_t gate[SHARE], up[SHARE];
#pragma unroll
                for (int cc = 0; cc < SHARE; cc += 32) {
                    tmem_ld32(lane_addr + c0 + cc, gate + cc);
                    tmem_ld32(lane_addr + BN / 2 + c0 + cc, up + cc);
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(drained);
                if (row < p.M) {
#pragma unroll
                    for (int j = 0; j < SHARE; j += 8) {
                        const int c = c0 + j;
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float g = round_to<__nv_bfloat16>(__uint_as_float(gate[j + e]));
                            const float u = round_to<__nv_bfloat16>(__uint_as_float(up[j + e]));
                            v[e] = round_to<__nv_bfloat16>(__fdividef(g, 1.f + __expf(-g))) * u;
                        }
                        if (n0 + c + 8 <= p.inter && (((uintptr_t)(out + c)) & 15) == 0) {
                            uint4 packed;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                            for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                            *reinterpret_cast<uint4*>(out + c) = packed;
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (n0 + c + e < p.inter) out[c + e] = __float2bfloat16_rn(v[e]);
                        }
                    }
                }
            } else {
                constexpr int SHARE = BN / 2;
                const int c0 = side * SHARE;
                uint32_t acc[SHARE];
#pragma unroll
                for (int cc = 0; cc < SHARE; cc += 32) tmem_ld32(lane_addr + c0 + cc, acc + cc);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(drained);
                if (row < p.M) {
#pragma unroll
                    for (int j = 0; j < SHARE; j += 8) {
                        const int c = c0 + j;
                        if (p.out_f32) {
                            float* out = (float*)p.y + (long long)row * p.ldy + n0 + c;
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (n0 + c + e < p.N) out[e] = __uint_as_float(acc[j + e]);
                        } else {
                            __nv_bfloat16* out = (__nv_bfloat16*)p.y + (long long)row * p.ldy + n0 + c;
                            if (n0 + c + 8 <= p.N && (((uintptr_t)out) & 15) == 0) {
                                uint4 v;
                                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    h[e] = __floats2bfloat162_rn(__uint_as_float(acc[j + 2 * e]), __uint_as_float(acc[j + 2 * e + 1]));
                                *reinterpret_cast<uint4*>(out) = v;
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    if (n0 + c + e < p.N) out[e] = __float2bfloat16_rn(__uint_as_float(acc[j + e]));
                            }
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    __syncwarp();
    pair_sync();                                     // neither CTA reads the other's shared memory or signals it any more
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

// A [rows, cols] row-major bfloat16 matrix, boxes of box_rows x 64 columns, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return ts_fail("gemm_tcgen05: the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ts_fail("gemm_tcgen05: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

bool g_pairing = true;

}  // namespace

// 0: every tile on one CTA.  1 (the default): large products run two CTAs a tile.
TS_API void ts_gemm_tcgen05_set_pairing(int enabled) { g_pairing = enabled != 0; }

// 1 if the sizes and addresses are ones TMA takes (16-byte aligned bases, row strides a multiple of 16 bytes).
TS_API int ts_gemm_tcgen05_supported(const void* W, const void* x, int M, int N, int K, long long ldx) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)W % 16 == 0) && ((uintptr_t)x % 16 == 0);
}

// y[M, N] = x[M, K] . W[N, K]^T (epilogue 0; out_dtype TS_BF16 or TS_F32), or y[M, N/2] = the SwiGLU of
// it with W = [gate rows | up rows] (epilogue 1, bfloat16 out).  `error` points to an int the host can
// read (0: fine; 1, 2, 3: a producer, MMA or epilogue wait ran out of time).
TS_API int ts_gemm_tcgen05(const void* W, const void* x, void* y, int M, int N, int K, long long ldx, long long ldy,
                           int epilogue, int out_dtype, int* error, cudaStream_t stream) {
    TS_REQUIRE(ts_gemm_tcgen05_supported(W, x, M, N, K, ldx), "gemm_tcgen05: sizes or alignment TMA does not take (M=%d N=%d K=%d)", M, N, K);
    TS_REQUIRE(error != nullptr, "gemm_tcgen05: an error word is needed");
    TS_REQUIRE(epilogue == EPI_STORE || epilogue == EPI_SWIGLU, "gemm_tcgen05: unknown epilogue %d", epilogue);
    TS_REQUIRE(out_dtype == TS_BF16 || (out_dtype == TS_F32 && epilogue == EPI_STORE), "gemm_tcgen05: unsupported output dtype");
    const int inter = N / 2;
    if (epilogue == EPI_SWIGLU) TS_REQUIRE(N % 2 == 0, "gemm_tcgen05: the SwiGLU epilogue needs gate and up halves (N=%d)", N);
    const int out_cols = epilogue == EPI_SWIGLU ? inter : N;
    const int m_tiles = (M + BM - 1) / BM;
    int sms = 148;
    int device = 0;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    // wide tiles halve the shared-memory traffic per flop; narrow ones when wide ones would leave SMs idle
    const int per_wide = epilogue == EPI_SWIGLU ? 128 : 256;
    const bool wide = (long long)m_tiles * ((out_cols + per_wide - 1) / per_wide) >= sms;
    const int bn = wide ? 256 : 128;
    const int out_per_tile = epilogue == EPI_SWIGLU ? bn / 2 : bn;
    const int num_tiles = m_tiles * ((out_cols + out_per_tile - 1) / out_per_tile);
    CUtensorMap map_a, map_b;
    GemmParams p{y, M, N, K, ldy, inter, out_dtype == TS_F32 ? 1 : 0, error};
    // Two CTAs a tile of 256 x 256 where every pair of SMs gets at least six such tiles: measured on a B200, pairs were
    // 1 to 3 % faster than single CTAs from there on (Llama 3.2 1B's gate/up product at 2,048 and 8,192 rows, Llama
    // 3.1 8B's from 1,024 rows) and the same or slower with fewer tiles, whose last round leaves more pairs idle.
    const int pair_cols = epilogue == EPI_SWIGLU ? 128 : 256;
    const long long pair_tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((out_cols + pair_cols - 1) / pair_cols);
    if (g_pairing && M > BM && pair_tiles >= 6 * (sms / 2)) {
        if (make_map(&map_a, x, M, K, ldx, BM)) return 1;
        if (make_map(&map_b, W, N, K, K, 128)) return 1;                 // each CTA loads half of a tile's rows of W
        const size_t pair_smem = (size_t)6 * (A_BYTES + 128 * BK * 2) + 1024;
        const int pairs = pair_tiles < sms / 2 ? (int)pair_tiles : sms / 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * pairs);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = pair_smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ts_chaining_enabled() ? 2 : 1;
        if (epilogue == EPI_SWIGLU) {
            cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair_smem);
            TS_CHAINED_CHECK("gemm_tcgen05", cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI_SWIGLU>, map_a, map_b, p));
        } else {
            cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair_smem);
            TS_CHAINED_CHECK("gemm_tcgen05", cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<EPI_STORE>, map_a, map_b, p));
        }
        return 0;
    }
    if (make_map(&map_a, x, M, K, ldx, BM)) return 1;
    if (make_map(&map_b, W, N, K, K, out_per_tile)) return 1;
    const bool deep = !wide && m_tiles == 1;
    const int stages = wide ? 4 : (deep ? 6 : 3);
    const size_t smem = (size_t)stages * (A_BYTES + bn * BK * 2) + 1024;
    const int slots = wide || deep ? sms : 2 * sms; // narrow tiles: half the shared memory and tensor memory each
    dim3 grid(num_tiles < slots ? num_tiles : slots);
#define TS_GEMM_LAUNCH(EPI_, BN_, STAGES_)                                                                 \
    do {                                                                                                   \
        auto kernel = gemm_tcgen05_kernel<EPI_, BN_, STAGES_>;                                             \
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
        TS_CHAINED_CHECK("gemm_tcgen05", launch_chained(kernel, grid, dim3(THREADS), smem, stream, map_a, map_b, p)); \
    } while (0)
    if (epilogue == EPI_SWIGLU) {
        if (wide) TS_GEMM_LAUNCH(EPI_SWIGLU, 256, 4);
        else if (deep) TS_GEMM_LAUNCH(EPI_SWIGLU, 128, 6);
        else TS_GEMM_LAUNCH(EPI_SWIGLU, 128, 3);
    } else {
        if (wide) TS_GEMM_LAUNCH(EPI_STORE, 256, 4);
        else if (deep) TS_GEMM_LAUNCH(EPI_STORE, 128, 6);
        else TS_GEMM_LAUNCH(EPI_STORE, 128, 3);
    }
#undef TS_GEMM_LAUNCH
    return 0;
}
