// y = x . W^T for a handful of rows of x (decode steps): bfloat16 inputs, float32 accumulation on
// tensor cores (mma.sync m16n8k16), output bfloat16 or float32.  The weight is the tall operand:
// a CTA takes 16 rows of W, its warps split K between them in blocks of 32, every thread streams W
// with 16-byte loads straight from global memory (each warp instruction reads 8 rows x 64 contiguous
// bytes), partial sums meet in shared memory in warp order.  The k indices inside a block of 32 are
// permuted the same way for both operands, so a thread's 8 contiguous weights and 8 contiguous
// activations feed two mma instructions without any shuffle.
//
// Epilogues: plain store, or SwiGLU: the CTA's 16 rows are 8 gate rows and the 8 up rows that belong
// to them, and it stores round(silu(gate)) * up (model/llama.py:80-83 of the reference).
//
// A third epilogue serves the q/k/v projection of decode steps: the CTA's 16 rows are 8 features of one
// head and their rotation partners half a head further on; it rotates q and k by the token's angles
// (model/llama.py:20-49 of the reference: rotate-half, float32), writes q to the output and k and v
// straight into the token's slot of the paged cache, which saves the separate rotary + store kernel.
//
// The split of K depends on N and K only, never on the number of rows of x, so a row's result does
// not depend on what else is in the batch.
//
// The weights' way onto the chip.  Every thread owns a ring of PJ slots in shared memory for its own
// fragments (the 16 bytes of row r and of row r + 8 of each of its k-blocks): cp.async copies k-block
// j into slot j % PJ, the thread reads it back into registers when its turn comes, and the slot is
// filled again with k-block j + PJ.  Nobody else reads a thread's slots, so there is no barrier and
// no bank conflict (a warp's slots are consecutive), and the copies in flight are bounded by shared
// memory, not by registers.  The ring is filled BEFORE the wait for the kernel ahead on the stream:
// the weights do not depend on that kernel, only x does, and where that kernel is a small one (a norm,
// the combination of the attention's splits) the memory is idle meanwhile, so that the q/k/v and
// output projections' whole matrices and a good third of the gate/up matrix are on the chip by the time
// x arrives.
#include "common.cuh"

namespace {

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ROPE = 2 };

// What the rotary + store epilogue needs.  Index data is written by the host before the step.
struct RopeArgs {
    const int* positions;        // [M]
    const int* seq_of_token;     // [M]; -1: a padding row (nothing is stored to the cache)
    const float* table;          // [positions][hd]: cos of the hd/2 angles, then sin; null: no rotation
    const int* block_table;      // [requests][table_width]
    int table_width;
    __nv_bfloat16* k_pool;
    __nv_bfloat16* v_pool;
    KVGeometry geo;
    int nh, nkv, hd, write_kv;
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
                 : "memory");
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {          // weights are read once: do not keep them in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <typename OUT>
__device__ __forceinline__ void store_out(OUT* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// MT: tiles of 8 rows of x; WARPS: warps per CTA (the split of K); UNROLL: k-blocks a warp has in
// flight per batch (two batches are in flight); MINB: CTAs per SM the register budget is held to;
// PJ: slots of each thread's ring of k-blocks in shared memory (a multiple of UNROLL): the copies in flight.
template <int MT, int WARPS, int EPI, typename OUT, int UNROLL, int MINB, int PJ>
__global__ void __launch_bounds__(WARPS * 32, MINB)
skinny_linear_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x, OUT* __restrict__ y,
                     int M, int N, int K, long long ldx, long long ldy, int inter, RopeArgs rope) {
    constexpr int ROWS = 16;                          // output rows of a CTA (8 pairs with the SwiGLU and rotary epilogues)
    __shared__ float partial[WARPS][MT][32][4];
    __shared__ float rope_cs[EPI == EPI_ROPE ? MT * 8 : 1][16];        // per token: 8 cos, 8 sin of this CTA's features
    __shared__ long long rope_slot[EPI == EPI_ROPE ? MT * 8 : 1];      // per token: offset of its slot in the pools, -1: none
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    // the rows of W this thread streams (fragment rows r and r + 8)
    long long row_lo, row_hi;
    int rows_valid;
    if (EPI == EPI_SWIGLU) {
        const int base = blockIdx.x * 8;
        rows_valid = min(8, inter - base);
        row_lo = base + min(r, rows_valid - 1);
        row_hi = (long long)inter + base + min(r, rows_valid - 1);
    } else if (EPI == EPI_ROPE) {
        const int blocks_per_head = rope.hd / 16;
        rows_valid = 8;
        row_lo = (long long)(blockIdx.x / blocks_per_head) * rope.hd + (blockIdx.x % blocks_per_head) * 8 + r;
        row_hi = row_lo + rope.hd / 2;
    } else {
        const int base = blockIdx.x * ROWS;
        rows_valid = min(ROWS, N - base);
        row_lo = base + min(r, rows_valid - 1);
        row_hi = base + min(r + 8, rows_valid - 1);
    }
    const __nv_bfloat16* w_lo = W + row_lo * K + c * 8;
    const __nv_bfloat16* w_hi = W + row_hi * K + c * 8;
    const __nv_bfloat16* x_row[MT];
    bool x_ok[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        const int token = t * 8 + r;
        x_ok[t] = token < M;
        x_row[t] = x + (long long)(x_ok[t] ? token : 0) * ldx + c * 8;
    }
    float acc[MT][4];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

    const int kblocks = K / 32;
    // The ring is filled before the kernel ahead on the stream has finished: the weights do not depend
    // on it.  x does, so it is read after chain_wait().
    extern __shared__ uint4 ring[];                   // [PJ][lo, hi][thread]
    constexpr int THREADS_ = WARPS * 32, GROUPS = PJ / UNROLL;
    // this warp's k-blocks are j = 0, 1, ...: kb = j * WARPS + warp; `blocks` of them exist
    const int blocks = warp < kblocks ? (kblocks - warp + WARPS - 1) / WARPS : 0;
    auto fill = [&](int j) {                          // k-block j into its slot; beyond the last one: nothing
        if (j < blocks) {
            const int kb = j * WARPS + warp;
            cp_async16(&ring[((j % PJ) * 2 + 0) * THREADS_ + threadIdx.x], w_lo + kb * 32);
            cp_async16(&ring[((j % PJ) * 2 + 1) * THREADS_ + threadIdx.x], w_hi + kb * 32);
        }
    };
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) fill(g * UNROLL + u);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    if (EPI == EPI_ROPE) {
        // the token's angles and its slot in the cache: index data, read while the first weights are on their way
        const int blocks_per_head = rope.hd / 16, head = blockIdx.x / blocks_per_head;
        const int j0 = (blockIdx.x % blocks_per_head) * 8, half = rope.hd / 2;
        for (int i = threadIdx.x; i < MT * 8 * 16; i += WARPS * 32) {
            const int token = i >> 4, e = i & 15;
            float v = e < 8 ? 1.f : 0.f;
            if (token < M && rope.table != nullptr && head < rope.nh + rope.nkv)
                v = rope.table[(long long)rope.positions[token] * rope.hd + (e < 8 ? j0 + e : half + j0 + e - 8)];
            rope_cs[token][e] = v;
        }
        for (int token = threadIdx.x; token < MT * 8; token += WARPS * 32) {
            long long slot = -1;
            if (token < M && rope.write_kv && head >= rope.nh) {
                const int seq = rope.seq_of_token[token];
                if (seq >= 0) {
                    const int pos = rope.positions[token];
                    const int page = rope.block_table[(long long)seq * rope.table_width + pos / rope.geo.page_tokens];
                    const int kvh = (head - rope.nh) % rope.nkv;
                    if (page >= 0 && page < rope.geo.num_pages)
                        slot = (long long)page * rope.geo.page_stride + rope.geo.entry_offset +
                               ((long long)kvh * rope.geo.page_tokens + pos % rope.geo.page_tokens) * rope.hd;
                }
            }
            rope_slot[token] = slot;
        }
    }
    chain_wait();
    chain_release();      // after the wait: letting later kernels in sooner (before it) slowed the step by a third
    // warp w takes the k-blocks w, w + WARPS, w + 2 WARPS, ... in that order whatever UNROLL and PJ are, so
    // a row's sum does not depend on the variant that the number of rows of x selects
    auto load_x = [&](uint4 (&xv)[UNROLL][MT], int j0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kb = min((j0 + u) * WARPS + warp, kblocks - 1);
#pragma unroll
            for (int t = 0; t < MT; ++t)
                xv[u][t] = x_ok[t] ? *reinterpret_cast<const uint4*>(x_row[t] + kb * 32) : make_uint4(0, 0, 0, 0);
        }
    };
    uint4 xv[UNROLL][MT], xn[UNROLL][MT];
    if (blocks > 0) load_x(xv, 0);
    for (int j0 = 0; j0 < blocks; j0 += UNROLL) {
        if (j0 + UNROLL < blocks) load_x(xn, j0 + UNROLL);           // the next batch of x is on its way under this one's products
        asm volatile("cp.async.wait_group %0;\n" ::"n"(GROUPS - 1) : "memory");   // this batch's copies have landed
        uint4 wl[UNROLL], wh[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            wl[u] = ring[(((j0 + u) % PJ) * 2 + 0) * THREADS_ + threadIdx.x];
            wh[u] = ring[(((j0 + u) % PJ) * 2 + 1) * THREADS_ + threadIdx.x];
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (j0 + u < blocks) {
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    mma_bf16(acc[t], wl[u].x, wh[u].x, wl[u].y, wh[u].y, xv[u][t].x, xv[u][t].y);
                    mma_bf16(acc[t], wl[u].z, wh[u].z, wl[u].w, wh[u].w, xv[u][t].z, xv[u][t].w);
                }
            }
        }
        // the slots just read are free (their values sit in registers the products above consumed): fill them again
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) fill(j0 + PJ + u);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int t = 0; t < MT; ++t) xv[u][t] = xn[u][t];
    }
    asm volatile("cp.async.wait_all;\n" ::: "memory");
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) partial[warp][t][lane][e] = acc[t][e];
    __syncthreads();
    // the warps' partial sums in warp order; thread (t, lane, e) owns row lane/4 (+8 for e >= 2), token t*8 + (lane%4)*2 + e%2
    if (EPI == EPI_SWIGLU) {
        for (int i = threadIdx.x; i < MT * 32 * 2; i += WARPS * 32) {
            const int t = i / 64, l = (i / 2) % 32, e = i % 2;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                gate += partial[w][t][l][e];
                up += partial[w][t][l][e + 2];
            }
            const int row = l >> 2, token = t * 8 + ((l & 3) << 1) + e;
            if (row < rows_valid && token < M) {
                // gate and up are materialised in bfloat16 by the reference before the activation
                const float g = round_to<__nv_bfloat16>(gate), u = round_to<__nv_bfloat16>(up);
                const float silu = round_to<__nv_bfloat16>(g / (1.f + expf(-g)));
                store_out<OUT>(y + (long long)token * ldy + blockIdx.x * 8 + row, silu * u);
            }
        }
    } else if (EPI == EPI_ROPE) {
        const int blocks_per_head = rope.hd / 16, head = blockIdx.x / blocks_per_head;
        const int j0 = (blockIdx.x % blocks_per_head) * 8, half = rope.hd / 2;
        for (int i = threadIdx.x; i < MT * 32 * 2; i += WARPS * 32) {
            const int t = i / 64, l = (i / 2) % 32, e = i % 2;
            float lo = 0.f, hi = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                lo += partial[w][t][l][e];
                hi += partial[w][t][l][e + 2];
            }
            const int row = l >> 2, token = t * 8 + ((l & 3) << 1) + e;
            if (token >= M) continue;
            // the projection is materialised in bfloat16 before the rotation, as in the reference
            const float x1 = round_to<__nv_bfloat16>(lo), x2 = round_to<__nv_bfloat16>(hi);
            const float cs = rope_cs[token][row], sn = rope_cs[token][8 + row];
            const float y1 = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));      // cos 1, sin 0 where nothing rotates
            const float y2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
            const int feature = head * rope.hd + j0 + row;
            if (head < rope.nh) {
                store_out<OUT>(y + (long long)token * ldy + feature, y1);
                store_out<OUT>(y + (long long)token * ldy + feature + half, y2);
            } else {
                const long long slot = rope_slot[token];
                if (slot >= 0) {
                    __nv_bfloat16* pool = head < rope.nh + rope.nkv ? rope.k_pool : rope.v_pool;
                    pool[slot + j0 + row] = __float2bfloat16_rn(y1);
                    pool[slot + j0 + row + half] = __float2bfloat16_rn(y2);
                }
            }
        }
    } else {
        constexpr int PER = 4;
        for (int i = threadIdx.x; i < MT * 32 * PER; i += WARPS * 32) {
            const int t = i / (32 * PER), l = (i / PER) % 32, e = i % PER;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += partial[w][t][l][e];
            const int row = (l >> 2) + ((e >> 1) << 3), token = t * 8 + ((l & 3) << 1) + (e & 1);
            if (row < rows_valid && token < M) store_out<OUT>(y + (long long)token * ldy + blockIdx.x * ROWS + row, v);
        }
    }
}

template <int MT, int WARPS, int EPI, typename OUT, int UNROLL, int MINB, int PJ>
int launch(const void* W, const void* x, void* y, int M, int N, int K, long long ldx, long long ldy, int inter,
           cudaStream_t stream, const RopeArgs& rope) {
    static_assert(PJ % UNROLL == 0 && PJ >= UNROLL, "the ring holds whole batches");
    const int tiles = EPI == EPI_SWIGLU ? (inter + 7) / 8 : (N + 15) / 16;
    const size_t staged = (size_t)PJ * 2 * WARPS * 32 * sizeof(uint4);
    auto kernel = skinny_linear_kernel<MT, WARPS, EPI, OUT, UNROLL, MINB, PJ>;
    if (staged > 32 * 1024) {
        static bool allowed = false;                   // per instantiation
        if (!allowed) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staged);
            if (e != cudaSuccess) return ts_fail("skinny_linear: cannot reserve %zu bytes of shared memory: %s", staged,
                                                 cudaGetErrorString(e));
            allowed = true;
        }
    }
    TS_CHAINED_CHECK("skinny_linear", launch_chained(kernel, dim3(tiles), dim3(WARPS * 32), staged, stream,
                                                     (const __nv_bfloat16*)W, (const __nv_bfloat16*)x, (OUT*)y, M, N, K, ldx,
                                                     ldy, inter, rope));
    return 0;
}

template <int WARPS, int EPI, typename OUT, int UNROLL, int MINB, int PJ>
int dispatch_m(const void* W, const void* x, void* y, int M, int N, int K, long long ldx, long long ldy, int inter,
               cudaStream_t stream, const RopeArgs& rope) {
    if (M <= 8) return launch<1, WARPS, EPI, OUT, UNROLL, MINB, PJ>(W, x, y, M, N, K, ldx, ldy, inter, stream, rope);
    if (M <= 16) return launch<2, WARPS, EPI, OUT, UNROLL, 1, PJ>(W, x, y, M, N, K, ldx, ldy, inter, stream, rope);
    // 32 rows of x with 16 warps: fewer loads in flight, to stay within the 128 registers a thread of 512 can have
    return launch<4, WARPS, EPI, OUT, (WARPS > 8 ? 2 : UNROLL), 1, PJ>(W, x, y, M, N, K, ldx, ldy, inter, stream, rope);
}

// How a product is cut into CTAs, chosen from N and K only (never from the rows of x).  Measured on
// a B200 with Llama 3.2 1B shapes (16 different weights in a row inside a CUDA graph, so nothing
// stays in L2): the aim is one wave of CTAs that covers all 148 SMs.
//   many row tiles (gate/up, vocabulary): 4 warps a tile, 7 CTAs per SM (1,036 slots);
//   149..296 tiles (q/k/v): 8 warps, 2 CTAs per SM;
//   up to 148 tiles (output projection, down): 16 warps, one CTA per SM.  (8-row tiles, twice the CTAs,
//   were no faster: the SMs that get two of them take as long as one 16-row tile.)
template <int EPI, typename OUT>
int dispatch_warps(const void* W, const void* x, void* y, int M, int N, int K, long long ldx, long long ldy, int inter,
                   cudaStream_t stream, const RopeArgs& rope = RopeArgs{}) {
    const int tiles = EPI == EPI_SWIGLU ? (inter + 7) / 8 : (N + 15) / 16;
    const int kblocks = K / 32;
    // Ring slots per thread (a k-block of a warp is 1 KB): 6 where seven CTAs share an SM (24 KB a CTA: over a third of a
    // 2,048-wide tile is on the chip before the wait), 8 where two CTAs or one do (a whole 2,048-wide tile).
    if (tiles > 296 || kblocks < 32)
        return dispatch_m<4, EPI, OUT, 2, 7, 6>(W, x, y, M, N, K, ldx, ldy, inter, stream, rope);
    if (tiles > 148) return dispatch_m<8, EPI, OUT, 4, 2, 8>(W, x, y, M, N, K, ldx, ldy, inter, stream, rope);
    return dispatch_m<16, EPI, OUT, 4, 1, 8>(W, x, y, M, N, K, ldx, ldy, inter, stream, rope);
}

}  // namespace

TS_API int ts_skinny_linear_max_rows() { return 32; }

// y[M, N] = x[M, K] . W[N, K]^T (epilogue 0), or y[M, N/2] = swiglu of it with W = [gate rows | up rows]
// (epilogue 1).  out_dtype: TS_BF16 or TS_F32.
TS_API int ts_skinny_linear(const void* W, const void* x, void* y, int M, int N, int K, long long ldx, long long ldy,
                            int epilogue, int out_dtype, cudaStream_t stream) {
    TS_REQUIRE(M >= 0 && N > 0 && K > 0, "skinny_linear: bad sizes M=%d N=%d K=%d", M, N, K);
    TS_REQUIRE(M <= ts_skinny_linear_max_rows(), "skinny_linear: %d rows of x; the kernel takes up to %d", M,
               ts_skinny_linear_max_rows());
    TS_REQUIRE(K % 32 == 0, "skinny_linear: K=%d is not a multiple of 32", K);
    TS_REQUIRE(ldx % 8 == 0, "skinny_linear: rows of x must start 16-byte aligned (stride %lld)", ldx);
    TS_REQUIRE(((uintptr_t)W % 16 == 0) && ((uintptr_t)x % 16 == 0), "skinny_linear: operands must be 16-byte aligned");
    if (M == 0) return 0;
    if (epilogue == EPI_SWIGLU) {
        TS_REQUIRE(N % 2 == 0, "skinny_linear: the SwiGLU epilogue needs gate and up halves (N=%d)", N);
        TS_REQUIRE(out_dtype == TS_BF16, "skinny_linear: the SwiGLU epilogue stores bfloat16");
        return dispatch_warps<EPI_SWIGLU, __nv_bfloat16>(W, x, y, M, N, K, ldx, ldy, N / 2, stream);
    }
    TS_REQUIRE(epilogue == EPI_STORE, "skinny_linear: unknown epilogue %d", epilogue);
    if (out_dtype == TS_BF16) return dispatch_warps<EPI_STORE, __nv_bfloat16>(W, x, y, M, N, K, ldx, ldy, 0, stream);
    if (out_dtype == TS_F32) return dispatch_warps<EPI_STORE, float>(W, x, y, M, N, K, ldx, ldy, 0, stream);
    return ts_fail("skinny_linear: unknown output dtype code %d", out_dtype);
}

// The q/k/v projection of a decode step with rotary embedding and the write into the paged cache in
// its epilogue: qkv[M, (nh + 2 nkv) hd] receives the rotated q (its k and v columns are not written);
// k (rotated) and v go to the slot of each token's position.  The rotary width must be the head
// size, a multiple of 16.  Pools are bfloat16, laid out as KVGeometry says.
TS_API int ts_skinny_qkv_rope_store(const void* W, const void* x, void* qkv, int M, int K, long long ldx,
                                    const int* positions, const int* seq_of_token, const float* table, int table_rows,
                                    int rot, const int* block_table, int table_width, void* k_pool, void* v_pool,
                                    long long page_stride, long long entry_offset, int page_tokens, int num_pages,
                                    int nh, int nkv, int hd, int write_kv, cudaStream_t stream) {
    TS_REQUIRE(M >= 0 && K > 0 && nh > 0 && nkv > 0 && hd > 0, "skinny_qkv_rope_store: bad sizes");
    TS_REQUIRE(M <= ts_skinny_linear_max_rows(), "skinny_qkv_rope_store: %d rows of x; the kernel takes up to %d", M,
               ts_skinny_linear_max_rows());
    TS_REQUIRE(K % 32 == 0, "skinny_qkv_rope_store: K=%d is not a multiple of 32", K);
    TS_REQUIRE(hd % 16 == 0, "skinny_qkv_rope_store: head size %d is not a multiple of 16", hd);
    TS_REQUIRE(table == nullptr || rot == hd, "skinny_qkv_rope_store: rotary width %d must equal the head size %d", rot, hd);
    TS_REQUIRE(table == nullptr || table_rows > 0, "skinny_qkv_rope_store: empty rotary table");
    TS_REQUIRE(ldx % 8 == 0 && ((uintptr_t)W % 16 == 0) && ((uintptr_t)x % 16 == 0),
               "skinny_qkv_rope_store: operands must be 16-byte aligned");
    TS_REQUIRE(page_tokens > 0 && num_pages > 0 && table_width > 0, "skinny_qkv_rope_store: bad cache geometry");
    if (M == 0) return 0;
    RopeArgs rope;
    rope.positions = positions;
    rope.seq_of_token = seq_of_token;
    rope.table = table;
    rope.block_table = block_table;
    rope.table_width = table_width;
    rope.k_pool = (__nv_bfloat16*)k_pool;
    rope.v_pool = (__nv_bfloat16*)v_pool;
    rope.geo = KVGeometry{page_stride, entry_offset, page_tokens, num_pages};
    rope.nh = nh;
    rope.nkv = nkv;
    rope.hd = hd;
    rope.write_kv = write_kv;
    const int N = (nh + 2 * nkv) * hd;
    return dispatch_warps<EPI_ROPE, __nv_bfloat16>(W, x, qkv, M, N, K, ldx, N, 0, stream, rope);
}
