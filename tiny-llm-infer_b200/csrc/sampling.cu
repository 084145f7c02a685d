// Sampling from float32 logits on the device: greedy, temperature and nucleus (top-p).
//
// The reference samples on the device with the Gumbel-max rule
// argmax_v(logit_v + temperature * -log(-log u_v)), temperature <= 1e-6 meaning plain
// argmax and ties going to the lower token id (kernels/src/sampling_kernel_cuda.cu:32-63),
// and applies top-p on the host by sorting the weights and keeping the smallest prefix
// whose sum reaches top_p * total (engine/src/llm_engine.cpp:110-145).  Here all three are
// one kernel.  The uniform u_v comes from a counter-based generator keyed by
// (row seed, token id), written out below, so that a draw does not depend on the batch a
// request is in and can be restated on the host.  The nucleus is found without a sort:
// a bisection on the weight threshold keeps the largest threshold whose kept mass still
// reaches top_p * total; tokens whose weights tie with the last kept one are all kept.
#include <cfloat>

#include "common.cuh"

namespace tllm {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Uniform in (0, 1): 23 random bits k -> (k + 0.5) / 2^23, exact in float32.
__host__ __device__ __forceinline__ float uniform_of(uint64_t seed, int token) {
    const uint64_t r = mix64(seed + 0x9E3779B97F4A7C15ull * (uint64_t)(token + 1));
    return ((float)(r >> 41) + 0.5f) * (1.0f / 8388608.0f);
}

struct Best {
    float value;
    int token;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    return (b.value > a.value || (b.value == a.value && b.token < a.token)) ? b : a;
}

__device__ __forceinline__ Best block_best(Best v, Best* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, v.value, o), __shfl_xor_sync(0xffffffffu, v.token, o)};
        v = better(v, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    Best r = (lane < nwarps) ? scratch[lane] : Best{-FLT_MAX, INT32_MAX};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, r.value, o), __shfl_xor_sync(0xffffffffu, r.token, o)};
        r = better(r, other);
    }
    return r;
}

// Two-stage form for greedy and temperature rows: `blocks_per_row` blocks share a row's
// vocabulary, each leaves its best candidate in `partial`, and a second small kernel picks
// among them (same comparison rule, so the result is that of the one-block form).  Rows
// with top_p < 1 are left to the one-block kernel below.
__global__ void sample_partial_kernel(const float* logits, int vocab, long long row_stride,
                                      const float* __restrict__ params,
                                      const unsigned long long* __restrict__ seeds,
                                      Best* __restrict__ partial, int blocks_per_row) {
    __shared__ Best best_scratch[32];
    TLLM_PDL_ENTER();
    const int row = blockIdx.y, b = blockIdx.x;
    const float temperature = params[2 * row], top_p = params[2 * row + 1];
    const bool greedy = !(temperature > 1.0e-6f);
    if (!greedy && top_p < 1.0f) return;
    const float* lg = logits + (size_t)row * row_stride;
    const uint64_t seed = seeds[row];
    const int chunk = (vocab + blocks_per_row - 1) / blocks_per_row;
    const int v0 = b * chunk, v1 = min(vocab, v0 + chunk);
    Best local{-FLT_MAX, INT32_MAX};
    if (greedy) {
        for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) local = better(local, Best{lg[v], v});
    } else {
        for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
            const float g = -logf(-logf(uniform_of(seed, v)));
            local = better(local, Best{lg[v] + temperature * g, v});
        }
    }
    local = block_best(local, best_scratch);
    if (threadIdx.x == 0) partial[(size_t)row * blocks_per_row + b] = local;
}

__global__ void sample_final_kernel(const Best* partial, int blocks_per_row,
                                    const float* __restrict__ params, int* __restrict__ out) {
    __shared__ Best best_scratch[32];
    TLLM_PDL_ENTER();
    const int row = blockIdx.x;
    const float temperature = params[2 * row], top_p = params[2 * row + 1];
    if (temperature > 1.0e-6f && top_p < 1.0f) return;
    Best local{-FLT_MAX, INT32_MAX};
    for (int b = threadIdx.x; b < blocks_per_row; b += blockDim.x)
        local = better(local, partial[(size_t)row * blocks_per_row + b]);
    local = block_best(local, best_scratch);
    if (threadIdx.x == 0) out[row] = local.token;
}

// One block per row.  params[row] = {temperature, top_p}; seeds[row] is the 64-bit key.
// With `only_nucleus` rows that are greedy or have top_p == 1 are skipped (the two-stage
// kernels above have done them).
__global__ void sample_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                              const float* __restrict__ params,
                              const unsigned long long* __restrict__ seeds, int* __restrict__ out,
                              int only_nucleus) {
    __shared__ Best best_scratch[32];
    __shared__ float sum_scratch[32];
    const int row = blockIdx.x;
    const float* lg = logits + (size_t)row * row_stride;
    const float temperature = params[2 * row], top_p = params[2 * row + 1];
    const uint64_t seed = seeds[row];
    const bool greedy = !(temperature > 1.0e-6f);
    if (only_nucleus && (greedy || !(top_p < 1.0f))) return;

    Best local{-FLT_MAX, INT32_MAX};
    if (greedy) {
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) local = better(local, Best{lg[v], v});
        local = block_best(local, best_scratch);
        if (threadIdx.x == 0) out[row] = local.token;
        return;
    }

    if (top_p < 1.0f) {
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) local = better(local, Best{lg[v], v});
        const float max_logit = block_best(local, best_scratch).value;
        const float inv_t = 1.0f / temperature;
        float z = 0.0f;
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) z += expf((lg[v] - max_logit) * inv_t);
        z = block_sum(z, sum_scratch);
        const float target = top_p * z;
        // weights w = exp((logit - max) / T) lie in (0, 1]; mass(w >= lo) >= target holds throughout
        float lo = 0.0f, hi = 1.0f + 1.0e-6f;
        for (int it = 0; it < 40; ++it) {
            const float mid = 0.5f * (lo + hi);
            float mass = 0.0f;
            for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
                const float w = expf((lg[v] - max_logit) * inv_t);
                if (w >= mid) mass += w;
            }
            mass = block_sum(mass, sum_scratch);
            if (mass >= target) lo = mid; else hi = mid;
        }
        // back from the weight threshold to a rule on the weights themselves
        local = Best{-FLT_MAX, INT32_MAX};
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
            const float w = expf((lg[v] - max_logit) * inv_t);
            if (w >= lo) {
                const float g = -logf(-logf(uniform_of(seed, v)));
                local = better(local, Best{lg[v] + temperature * g, v});
            }
        }
        local = block_best(local, best_scratch);
        if (threadIdx.x == 0) out[row] = local.token;
        return;
    }
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
        const float g = -logf(-logf(uniform_of(seed, v)));
        local = better(local, Best{lg[v] + temperature * g, v});
    }
    local = block_best(local, best_scratch);
    if (threadIdx.x == 0) out[row] = local.token;
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_sample(const float* logits, int rows, int vocab, long long row_stride,
                           const float* params, const unsigned long long* seeds, int* out,
                           cudaStream_t stream) {
    TLLM_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes");
    if (rows == 0) return 0;
    const int block = vocab >= 8192 ? 1024 : 256;
    sample_kernel<<<rows, block, 0, stream>>>(logits, vocab, row_stride, params, seeds, out, 0);
    return finish_launch("sample");
}

// The same result with the vocabulary of a row shared by `blocks_per_row` blocks.
// `partial` is scratch of rows * blocks_per_row * 8 bytes.  `any_nucleus` tells whether some
// row has temperature > 1e-6 and top_p < 1 (those rows need the one-block kernel).
extern "C" int tllm_sample_split(const float* logits, int rows, int vocab, long long row_stride,
                                 const float* params, const unsigned long long* seeds, int* out,
                                 void* partial, int blocks_per_row, int any_nucleus, cudaStream_t stream) {
    TLLM_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes");
    TLLM_REQUIRE(partial != nullptr && blocks_per_row >= 1 && blocks_per_row <= 1024 && rows <= 65535,
                 "sample: bad split");
    if (rows == 0) return 0;
    launch_pdl(kPdlOther, sample_partial_kernel, dim3(blocks_per_row, rows), dim3(256), 0, stream,
        logits, vocab, row_stride, params, seeds, (Best*)partial, blocks_per_row);
    int rc = finish_launch("sample_partial");
    if (rc) return rc;
    launch_pdl(kPdlOther, sample_final_kernel, dim3(rows), dim3(64), 0, stream, (const Best*)partial, blocks_per_row, params, out);
    rc = finish_launch("sample_final");
    if (rc || !any_nucleus) return rc;
    sample_kernel<<<rows, vocab >= 8192 ? 1024 : 256, 0, stream>>>(logits, vocab, row_stride, params, seeds, out, 1);
    return finish_launch("sample");
}

// The generator, for host-side restatements in tests.
extern "C" float tllm_uniform_of(unsigned long long seed, int token) { return uniform_of(seed, token); }
