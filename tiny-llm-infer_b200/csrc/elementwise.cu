// Embedding gather, residual-add + RMSNorm, SwiGLU and storage-type conversion.
//
// What the reference does with separate launches (embed_kernel_cuda.cu:6-28,
// add_kernel_cuda.cu:7-14 followed by rmsnorm_kernel_cuda.cu:8-39,
// swiglu_kernel_cuda.cu:7-27) is fused here around one rule: the residual stream is
// a float32 tensor that only this file's kernels write, so the residual sum and the
// norm's mean are 32-bit in both storage modes.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace tllm {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int finish_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] widened to float32.  Rows with ids[t] < 0 (padding of a
// fixed-size batch) become zero.  Ids are range-checked on the host; the clamp below
// only keeps a faulty caller from reading outside the table.
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab) {
    const int t = blockIdx.x;
    int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    if (id >= vocab) id = vocab - 1;
    const TW* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<TW>(src[i]);
}

// ---------------------------------------------------------------- add + RMSNorm
// v = h[r, :] (+ delta[r, :]);  out[o, :] = gain * v / sqrt(mean(v^2) + eps).
// Without `rows`: r = o = blockIdx.x and v is written back to h (the residual sum).
// With `rows`: r = rows[o], h is left as it is (used for the last norm, on the rows
// whose logits are wanted).  gain is read as float32 or bfloat16.
template <typename TD, typename TG, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const TG* __restrict__ gain, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows,
                                   int width) {
    __shared__ float scratch[32];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    if (r < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_f32<TO>(0.0f);
        return;
    }
    float* hr = h + (size_t)r * width;
    const TD* dr = delta ? delta + (size_t)r * width : nullptr;
    const bool write_back = (rows == nullptr) && (dr != nullptr);
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = hr[i];
        if (dr) v += to_f32<TD>(dr[i]);
        if (write_back) hr[i] = v;
        sum += v * v;
    }
    sum = block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = hr[i];                       // already holds the sum when written back
        if (dr && !write_back) v += to_f32<TD>(dr[i]);
        dst[i] = from_f32<TO>(to_f32<TG>(gain[i]) * v * scale);
    }
}

// ---------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i], silu(x) = x / (1 + exp(-x)), in float32.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                              size_t total) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / inter, i = idx - t * inter;
        const float g = to_f32<T>(gu[t * 2 * inter + i]);
        const float u = to_f32<T>(gu[t * 2 * inter + inter + i]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

template <typename TS, typename TD>
__global__ void cast_kernel(const TS* __restrict__ src, TD* __restrict__ dst, size_t n) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < n; idx += stride) dst[idx] = from_f32<TD>(to_f32<TS>(src[idx]));
}

static int grid_for(size_t total, int block) {
    size_t g = (total + block - 1) / block;
    const size_t cap = 148 * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* h, const void* delta, const void* gain, int gain_dtype,
                              float eps, void* out, const int* rows, int n_out, int width,
                              cudaStream_t stream) {
    const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (gain_dtype == kBF16)
        add_rmsnorm_kernel<TD, bf16, TO><<<n_out, block, 0, stream>>>(
            h, (const TD*)delta, (const bf16*)gain, eps, (TO*)out, rows, width);
    else
        add_rmsnorm_kernel<TD, float, TO><<<n_out, block, 0, stream>>>(
            h, (const TD*)delta, (const float*)gain, eps, (TO*)out, rows, width);
    return finish_launch("add_rmsnorm");
}

}  // namespace tllm

using namespace tllm;

extern "C" {

const char* tllm_last_error() { return g_error; }

int tllm_embedding(const int* ids, const void* table, int table_dtype, float* out, int tokens,
                   int hidden, int vocab, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
    if (tokens == 0) return 0;
    const int block = hidden >= 1024 ? 256 : 128;
    if (table_dtype == kBF16)
        embedding_kernel<bf16><<<tokens, block, 0, stream>>>(ids, (const bf16*)table, out, hidden, vocab);
    else if (table_dtype == kF32)
        embedding_kernel<float><<<tokens, block, 0, stream>>>(ids, (const float*)table, out, hidden, vocab);
    else
        TLLM_REQUIRE(false, "embedding: unknown dtype %d", table_dtype);
    return finish_launch("embedding");
}

// act_dtype is the storage type of both `delta` and `out`.
int tllm_add_rmsnorm(float* h, const void* delta, const void* gain, int gain_dtype, float eps,
                     void* out, int act_dtype, const int* rows, int n_out, int width,
                     cudaStream_t stream) {
    TLLM_REQUIRE(n_out >= 0 && width > 0, "add_rmsnorm: bad sizes");
    TLLM_REQUIRE(gain_dtype == kBF16 || gain_dtype == kF32, "add_rmsnorm: unknown gain dtype");
    TLLM_REQUIRE(eps > 0.0f, "add_rmsnorm: eps must be positive");
    if (n_out == 0) return 0;
    if (act_dtype == kBF16)
        return launch_add_rmsnorm<bf16, bf16>(h, delta, gain, gain_dtype, eps, out, rows, n_out, width, stream);
    if (act_dtype == kF32)
        return launch_add_rmsnorm<float, float>(h, delta, gain, gain_dtype, eps, out, rows, n_out, width, stream);
    TLLM_REQUIRE(false, "add_rmsnorm: unknown dtype %d", act_dtype);
}

int tllm_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter,
                cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && inter > 0, "swiglu: bad sizes");
    const size_t total = (size_t)tokens * inter;
    if (total == 0) return 0;
    const int block = 256, grid = grid_for(total, block);
    if (dtype == kBF16)
        swiglu_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)gate_up, (bf16*)out, inter, total);
    else if (dtype == kF32)
        swiglu_kernel<float><<<grid, block, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
    else
        TLLM_REQUIRE(false, "swiglu: unknown dtype %d", dtype);
    return finish_launch("swiglu");
}

int tllm_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
              cudaStream_t stream) {
    TLLM_REQUIRE(n >= 0, "cast: bad size");
    if (n == 0) return 0;
    const int block = 256, grid = grid_for((size_t)n, block);
    if (src_dtype == kBF16 && dst_dtype == kF32)
        cast_kernel<bf16, float><<<grid, block, 0, stream>>>((const bf16*)src, (float*)dst, (size_t)n);
    else if (src_dtype == kF32 && dst_dtype == kBF16)
        cast_kernel<float, bf16><<<grid, block, 0, stream>>>((const float*)src, (bf16*)dst, (size_t)n);
    else
        TLLM_REQUIRE(false, "cast: unsupported pair %d -> %d", src_dtype, dst_dtype);
    return finish_launch("cast");
}

}  // extern "C"
