// y[M, N] = x[M, K] . W[N, K]^T, the plain way: one thread per output element, the sum over k
// in order in float32 (fused multiply-add), inputs of either storage type widened exactly.
// No tiles, no tensor cores, no shared memory: it is the kernel the fast products (the
// weight-streaming one, the tcgen05 one, the library's) are checked against in the tests, at
// sizes a float64 product on the host would take too long for, and it takes every size.
//
// The reference's counterpart is its CPU product (kernels/src/matmul_kernel_cpu.cpp:6-36: a loop
// over k per output with a float32 sum), which plays the same part beside cublasHgemm.
#include "common.cuh"

namespace tllm {

template <typename TX, typename TW, typename TY>
__global__ void gemm_plain_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y,
                                  int M, int N, int K) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)M * N) return;
    const int m = (int)(idx / N), n = (int)(idx - (long long)m * N);
    const TX* xr = x + (size_t)m * K;
    const TW* wr = w + (size_t)n * K;
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) acc = fmaf(to_f32<TX>(xr[k]), to_f32<TW>(wr[k]), acc);
    y[idx] = from_f32<TY>(acc);
}

template <typename TX, typename TW>
static int launch_plain(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K, cudaStream_t stream) {
    const long long total = (long long)M * N;
    const int block = 256;
    const long long grid = (total + block - 1) / block;
    TLLM_REQUIRE(grid <= 0x7fffffffLL, "gemm_plain: %lld outputs are too many for one launch", total);
    if (y_dtype == kF32)
        gemm_plain_kernel<TX, TW, float><<<(unsigned)grid, block, 0, stream>>>((const TX*)x, (const TW*)w, (float*)y, M, N, K);
    else
        gemm_plain_kernel<TX, TW, bf16><<<(unsigned)grid, block, 0, stream>>>((const TX*)x, (const TW*)w, (bf16*)y, M, N, K);
    return finish_launch("gemm_plain");
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_gemm_plain(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                               int M, int N, int K, cudaStream_t stream) {
    TLLM_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_plain: bad sizes");
    const auto known = [](int d) { return d == kF32 || d == kBF16; };
    TLLM_REQUIRE(known(x_dtype) && known(w_dtype) && known(y_dtype), "gemm_plain: unknown dtype");
    if (M == 0) return 0;
    if (x_dtype == kF32)
        return w_dtype == kF32 ? launch_plain<float, float>(x, w, y, y_dtype, M, N, K, stream)
                               : launch_plain<float, bf16>(x, w, y, y_dtype, M, N, K, stream);
    return w_dtype == kF32 ? launch_plain<bf16, float>(x, w, y, y_dtype, M, N, K, stream)
                           : launch_plain<bf16, bf16>(x, w, y, y_dtype, M, N, K, stream);
}
