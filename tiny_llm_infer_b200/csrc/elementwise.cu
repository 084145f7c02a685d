// Embedding gather, residual-add + RMSNorm, SwiGLU and storage-type conversion.
//
// What the reference does with separate launches (embed_kernel_cuda.cu:6-28,
// add_kernel_cuda.cu:7-14 followed by rmsnorm_kernel_cuda.cu:8-39,
// swiglu_kernel_cuda.cu:7-27) is fused here around one rule: the residual stream is
// a float32 tensor that only this file's kernels write, so the residual sum and the
// norm's mean are 32-bit in both storage modes.
//
// Pointers to what an earlier kernel of the step has written carry no __restrict__: with
// programmatic dependent launch this kernel may start before that kernel ends, and the
// read-only load path the compiler would otherwise choose may then return stale data.
//
// Every kernel has a vector form (16-byte loads and stores, eight elements per thread per
// access, every load of a row issued before the first dependent instruction) for widths that
// are multiples of eight, and a scalar form that takes any width.
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

// ---------------------------------------------------------------- 8-element accesses
template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Vec8<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] widened to float32.  Rows with ids[t] < 0 (padding of a
// fixed-size batch) become zero.  Ids are range-checked on the host; the clamp below
// only keeps a faulty caller from reading outside the table.
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab) {
    TLLM_PDL_ENTER();
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

template <typename TW>
__global__ void embedding_vec_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                     float* __restrict__ out, int hidden, int vocab) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    const bool pad = id < 0;
    if (id >= vocab) id = vocab - 1;
    const TW* src = table + (size_t)(pad ? 0 : id) * hidden;
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (!pad) Vec8<TW>::load(src + c * 8, v);
        Vec8<float>::store(dst + c * 8, v);
    }
}

// ---------------------------------------------------------------- add + RMSNorm
// v = h[r, :] (+ delta[r, :]);  out[o, :] = gain * v / sqrt(mean(v^2) + eps).
// Without `rows`: r = o = blockIdx.x and v is written back to h (the residual sum).
// With `rows`: r = rows[o], h is left as it is (used for the last norm, on the rows
// whose logits are wanted).  gain is read as float32 or bfloat16.
template <typename TD, typename TG, typename TO>
__global__ void add_rmsnorm_kernel(float* h, const TD* delta,
                                   const TG* __restrict__ gain, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows,
                                   int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
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

// Vector form: the row lives in registers between the sum and the scaling, CHUNKS groups of
// eight elements per thread (width <= blockDim * 8 * CHUNKS, width a multiple of 8).
template <typename TD, typename TG, typename TO, int CHUNKS>
__global__ void add_rmsnorm_vec_kernel(float* h, const TD* delta,
                                       const TG* __restrict__ gain, float eps, TO* __restrict__ out,
                                       const int* __restrict__ rows, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    const int n_chunks = width >> 3;
    if (r < 0) {
        const float zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) Vec8<TO>::store(dst + c * 8, zero);
        return;
    }
    float* hr = h + (size_t)r * width;
    const TD* dr = delta ? delta + (size_t)r * width : nullptr;
    const bool write_back = (rows == nullptr) && (dr != nullptr);
    float v[CHUNKS][8], d[CHUNKS][8];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            Vec8<float>::load(hr + c * 8, v[j]);
            if (dr) Vec8<TD>::load(dr + c * 8, d[j]);
        }
    }
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (dr) v[j][e] += d[j][e];
                sum += v[j][e] * v[j][e];
            }
            if (write_back) Vec8<float>::store(hr + c * 8, v[j]);
        }
    }
    sum = block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / (float)width + eps);
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            float g[8];
            Vec8<TG>::load(gain + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = g[e] * v[j][e] * scale;
            Vec8<TO>::store(dst + c * 8, g);
        }
    }
}

// ---------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gate) * up, silu(x) = x / (1 + exp(-x)), in float32.  Stacked columns: gate at
// gu[t, i], up at gu[t, inter + i].  Interleaved by eight: columns come in groups of sixteen,
// eight gates followed by their eight ups, so gate at gu[t, 16 (i / 8) + i % 8] and up 8 further.
template <typename T>
__global__ void swiglu_kernel(const T* gu, T* out, int inter, int interleaved,
                              size_t total) {
    TLLM_PDL_ENTER();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / inter, i = idx - t * inter;
        const size_t gi = interleaved ? 16 * (i >> 3) + (i & 7) : i, ui = interleaved ? gi + 8 : inter + i;
        const float g = to_f32<T>(gu[t * 2 * inter + gi]);
        const float u = to_f32<T>(gu[t * 2 * inter + ui]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

template <typename T>
__global__ void swiglu_vec_kernel(const T* gu, T* out, int inter, int interleaved,
                                  size_t total_chunks) {
    TLLM_PDL_ENTER();
    const int per_row = inter >> 3;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total_chunks; idx += stride) {
        const size_t t = idx / per_row, c = idx - t * per_row;
        float g[8], u[8];
        Vec8<T>::load(gu + t * 2 * inter + (interleaved ? c * 16 : c * 8), g);
        Vec8<T>::load(gu + t * 2 * inter + (interleaved ? c * 16 + 8 : inter + c * 8), u);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = g[e] / (1.0f + expf(-g[e])) * u[e];
        Vec8<T>::store(out + t * inter + c * 8, g);
    }
}

__global__ void feed_tokens_kernel(int* ids, const int* places, const int* rows, const int* sampled, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[places[i]] = sampled[rows[i]];
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

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename TD, typename TG, typename TO>
static int launch_add_rmsnorm_typed(float* h, const void* delta, const void* gain, float eps, void* out,
                                    const int* rows, int n_out, int width, cudaStream_t stream) {
    const bool vec = width % 8 == 0 && aligned16(h) && aligned16(delta) && aligned16(gain) && aligned16(out);
    const int chunks = width / 8;
    if (vec && chunks <= 1024 * 4) {
        int block = 64;
        while (block < 1024 && block < chunks) block *= 2;
        const int per_thread = (chunks + block - 1) / block;
#define VEC_LAUNCH(C)                                                                 \
    launch_pdl(kPdlNorm, add_rmsnorm_vec_kernel<TD, TG, TO, C>, dim3(n_out), dim3(block), 0, stream, \
               h, (const TD*)delta, (const TG*)gain, eps, (TO*)out, rows, width)
        if (per_thread <= 1) VEC_LAUNCH(1);
        else if (per_thread <= 2) VEC_LAUNCH(2);
        else VEC_LAUNCH(4);
#undef VEC_LAUNCH
    } else {
        const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
        launch_pdl(kPdlNorm, add_rmsnorm_kernel<TD, TG, TO>, dim3(n_out), dim3(block), 0, stream,
                   h, (const TD*)delta, (const TG*)gain, eps, (TO*)out, rows, width);
    }
    return finish_launch("add_rmsnorm");
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* h, const void* delta, const void* gain, int gain_dtype,
                              float eps, void* out, const int* rows, int n_out, int width,
                              cudaStream_t stream) {
    if (gain_dtype == kBF16)
        return launch_add_rmsnorm_typed<TD, bf16, TO>(h, delta, gain, eps, out, rows, n_out, width, stream);
    return launch_add_rmsnorm_typed<TD, float, TO>(h, delta, gain, eps, out, rows, n_out, width, stream);
}

}  // namespace tllm

using namespace tllm;

extern "C" {

const char* tllm_last_error() { return g_error; }

int tllm_embedding(const int* ids, const void* table, int table_dtype, float* out, int tokens,
                   int hidden, int vocab, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
    TLLM_REQUIRE(table_dtype == kBF16 || table_dtype == kF32, "embedding: unknown dtype %d", table_dtype);
    if (tokens == 0) return 0;
    const bool vec = hidden % 8 == 0 && aligned16(table) && aligned16(out);
    const int block = vec ? (hidden >= 2048 ? 256 : 128) : (hidden >= 1024 ? 256 : 128);
    if (table_dtype == kBF16) {
        if (vec) launch_pdl(kPdlOther, embedding_vec_kernel<bf16>, dim3(tokens), dim3(block), 0, stream, ids, (const bf16*)table, out, hidden, vocab);
        else launch_pdl(kPdlOther, embedding_kernel<bf16>, dim3(tokens), dim3(block), 0, stream, ids, (const bf16*)table, out, hidden, vocab);
    } else {
        if (vec) launch_pdl(kPdlOther, embedding_vec_kernel<float>, dim3(tokens), dim3(block), 0, stream, ids, (const float*)table, out, hidden, vocab);
        else launch_pdl(kPdlOther, embedding_kernel<float>, dim3(tokens), dim3(block), 0, stream, ids, (const float*)table, out, hidden, vocab);
    }
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

int tllm_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter, int interleaved,
                cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && inter > 0, "swiglu: bad sizes");
    TLLM_REQUIRE(!interleaved || inter % 8 == 0, "swiglu: interleaved columns need a multiple of 8, not %d", inter);
    TLLM_REQUIRE(dtype == kBF16 || dtype == kF32, "swiglu: unknown dtype %d", dtype);
    const size_t total = (size_t)tokens * inter;
    if (total == 0) return 0;
    const int block = 256;
    if (inter % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
        const size_t chunks = total / 8;
        const int grid = grid_for(chunks, block);
        if (dtype == kBF16)
            launch_pdl(kPdlSwiglu, swiglu_vec_kernel<bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, interleaved, chunks);
        else
            launch_pdl(kPdlSwiglu, swiglu_vec_kernel<float>, dim3(grid), dim3(block), 0, stream, (const float*)gate_up, (float*)out, inter, interleaved, chunks);
    } else {
        const int grid = grid_for(total, block);
        if (dtype == kBF16)
            launch_pdl(kPdlSwiglu, swiglu_kernel<bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, interleaved, total);
        else
            launch_pdl(kPdlSwiglu, swiglu_kernel<float>, dim3(grid), dim3(block), 0, stream, (const float*)gate_up, (float*)out, inter, interleaved, total);
    }
    return finish_launch("swiglu");
}

// ids[places[i]] = sampled[rows[i]] for i < n: tokens that a step still being sampled from gives
// the next step, without the host in between.  All four are device arrays of int32.
int tllm_feed_tokens(int* ids, const int* places, const int* rows, const int* sampled, int n, cudaStream_t stream) {
    TLLM_REQUIRE(n >= 0 && ids && places && rows && sampled, "feed_tokens: bad arguments");
    if (n == 0) return 0;
    feed_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, places, rows, sampled, n);
    return finish_launch("feed_tokens");
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
