// A kernel that belongs to a toy part defined in tests/test_toy_parts.py, not to the engine: the test
// compiles it as an extension of the kernel library and calls it through Ops.call, to show that a part
// can bring CUDA code of its own without a change to the framework's files.
#include "common.cuh"

namespace {

// out[r, c] = x[r, c] * gain[c] + shift   (float32)
__global__ void toy_gain_kernel(const float* x, const float* gain, float shift, float* out, int rows, int cols) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < (long long)rows * cols) out[i] = x[i] * gain[i % cols] + shift;
}

}  // namespace

TS_API int toy_gain(const void* x, const void* gain, float shift, void* out, int rows, int cols, cudaStream_t stream) {
    TS_REQUIRE(rows >= 0 && cols > 0, "toy_gain: bad sizes %d x %d", rows, cols);
    if (rows == 0) return 0;
    const long long n = (long long)rows * cols;
    toy_gain_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const float*)x, (const float*)gain, shift,
                                                                     (float*)out, rows, cols);
    TS_LAUNCH_CHECK("toy_gain");
    return 0;
}
