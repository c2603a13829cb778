// float32 matrix product C[M, N] = A[M, K] . B[N, K]^T with FFMA and float32 accumulation: the
// engine's true 32-bit projection (no tensor-core mode that rounds its inputs).  Each output element
// sums over k in ascending order, so a row's result does not depend on what else is in the batch.
// Any M, N, K; rows of A and B are K-contiguous (the checkpoint's [out_features, in_features]).
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                long long lda, long long ldb, long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const int tr = (tid / 16) * TM, tc = (tid % 16) * TN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    const int lk = tid % BK, lr = tid / BK;               // each thread loads 4 rows at column lk
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < BM / 16; ++i) {
            const int r = lr + 16 * i;
            const int gr = row0 + r, gk = k0 + lk;
            As[lk][r] = (gr < M && gk < K) ? A[(long long)gr * lda + gk] : 0.f;
            const int gc = col0 + r;
            Bs[lk][r] = (gc < N && gk < K) ? B[(long long)gc * ldb + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][tr + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[k][tc + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gr = row0 + tr + i;
        if (gr >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gc = col0 + tc + j;
            if (gc < N) C[(long long)gr * ldc + gc] = acc[i][j];
        }
    }
}

TS_API int ts_sgemm_nt(const float* A, const float* B, float* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, cudaStream_t stream) {
    TS_REQUIRE(M >= 0 && N > 0 && K > 0, "sgemm: bad sizes M=%d N=%d K=%d", M, N, K);
    TS_REQUIRE(lda >= K && ldb >= K && ldc >= N, "sgemm: row strides smaller than the rows");
    if (M == 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    TS_REQUIRE(grid.y <= 65535, "sgemm: M=%d needs more than 65535 row tiles", M);
    sgemm_nt_kernel<<<grid, 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc);
    TS_LAUNCH_CHECK("sgemm");
    return 0;
}
