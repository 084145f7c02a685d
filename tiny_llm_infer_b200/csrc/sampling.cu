// Sampling from float32 logits on the device: greedy, temperature and nucleus (top-p).
//
// The reference samples on the device with the Gumbel-max rule
// argmax_v(logit_v + temperature * -log(-log u_v)), temperature <= 1e-6 meaning plain
// argmax and ties going to the lower token id (kernels/src/sampling_kernel_cuda.cu:32-63),
// and applies top-p on the host by sorting the weights and keeping the smallest prefix
// whose sum reaches top_p * total (engine/src/llm_engine.cpp:110-145).  Here all three are
// one kernel.  The uniform u_v comes from a counter-based generator keyed by
// (row seed, token id), written out below, so that a draw does not depend on the batch a
// request is in and can be restated on the host.  The nucleus is found without a sort, by a
// radix selection: with t = (max - logit) / T >= 0 a token's weight is e^-t, and the
// nucleus is {t <= t*} for the smallest t* whose kept mass reaches top_p * total.  t is
// cut to a 33-bit fixed-point key (2^-28 steps below 32; weights under e^-32 of the largest
// carry no mass), and three passes over the row, each a histogram of mass over 2048 bins
// of the next 11 key bits, find the key of t*.  Mass is summed in 2^-40 fixed point in
// 64-bit integers, so the sums do not depend on the order in which threads add and the
// same logits give the same nucleus on every run.  Tokens whose keys tie with the last
// kept one are all kept.
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

// ---- nucleus by radix selection (one block per row; blockDim.x divides kNucleusBins) ----
constexpr int kNucleusBits = 11, kNucleusBins = 1 << kNucleusBits, kNucleusLevels = 3;
constexpr unsigned long long kNucleusFarKey = (1ull << (kNucleusBits * kNucleusLevels)) - 1;

// t >= 0 in 2^-28 steps; everything from 32 on (and NaN) shares the last key.
__device__ __forceinline__ unsigned long long nucleus_key(float t) {
    return t < 32.0f ? (unsigned long long)(t * 268435456.0f) : kNucleusFarKey;
}

// e^-t in 2^-40 fixed point; keys at or beyond 32 weigh nothing.
__device__ __forceinline__ unsigned long long nucleus_mass(float t) {
    return t < 32.0f ? __float2ull_rn(expf(-t) * 1099511627776.0f) : 0ull;
}

__device__ __forceinline__ unsigned long long warp_scan_u64(unsigned long long v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += up;
    }
    return v;
}

// hist[kNucleusBins] holds mass per bin.  Returns the total; `before` becomes the mass of
// the bins ahead of this thread's own (a contiguous run of kNucleusBins / blockDim.x bins)
// and `own` the mass of that run.
__device__ __forceinline__ unsigned long long nucleus_scan(const unsigned long long* hist,
                                                           unsigned long long* scan,
                                                           unsigned long long& before,
                                                           unsigned long long& own) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int per = kNucleusBins / blockDim.x;
    own = 0;
    for (int i = 0; i < per; ++i) own += hist[threadIdx.x * per + i];
    const unsigned long long incl = warp_scan_u64(own, lane);
    if (lane == 31) scan[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const unsigned long long total = lane < nwarps ? scan[lane] : 0ull;
        const unsigned long long through = warp_scan_u64(total, lane);
        scan[lane] = through - total;               // mass of the warps ahead
        if (lane == 31) scan[32] = through;
    }
    __syncthreads();
    before = scan[warp] + incl - own;
    return scan[32];
}

// The key of the last token of the nucleus: the smallest key whose kept mass (all keys up
// to it) reaches top_p * total.
__device__ unsigned long long nucleus_last_key(const float* lg, int vocab, float max_logit, float inv_t,
                                               float top_p, unsigned long long* hist,
                                               unsigned long long* scan) {
    unsigned long long prefix = 0, target = 0;      // key bits settled so far; mass still to find
    for (int level = 0; level < kNucleusLevels; ++level) {
        const int shift = kNucleusBits * (kNucleusLevels - 1 - level);
        for (int i = threadIdx.x; i < kNucleusBins; i += blockDim.x) hist[i] = 0ull;
        if (threadIdx.x == 0) {                      // what stands if no mass is found at all
            scan[33] = kNucleusBins - 1;
            scan[34] = 0ull;
        }
        __syncthreads();
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
            const float t = (max_logit - lg[v]) * inv_t;
            const unsigned long long key = nucleus_key(t);
            if (level == 0 || (key >> (shift + kNucleusBits)) == prefix) {
                const unsigned long long m = nucleus_mass(t);
                if (m) atomicAdd(&hist[(key >> shift) & (kNucleusBins - 1)], m);
            }
        }
        __syncthreads();
        unsigned long long before, own;
        const unsigned long long total = nucleus_scan(hist, scan, before, own);
        if (level == 0) {
            target = (unsigned long long)((double)top_p * (double)total);
            if (target < 1ull) target = 1ull;
            if (target > total) target = total;
        }
        if (before < target && target <= before + own) {   // exactly one thread: sums never fall
            const int per = kNucleusBins / blockDim.x;
            int bin = threadIdx.x * per;
            unsigned long long run = before;
            while (run + hist[bin] < target) run += hist[bin++];
            scan[33] = (unsigned long long)bin;
            scan[34] = target - run;                 // what the chosen bin still has to give
        }
        __syncthreads();
        prefix = (prefix << kNucleusBits) | scan[33];
        target = scan[34];
        __syncthreads();
    }
    return prefix;
}

// Two-stage form: `blocks_per_row` blocks share a row's vocabulary, each leaves its best
// candidate in `partial`, and a second small kernel picks among them (same comparison rule,
// so the result is that of the one-block form).  For a row with top_p < 1 the candidate is
// the block's largest logit, which the nucleus passes below start from, and the blocks clear
// the row's histograms (`hist`, null when no row has top_p < 1).
__global__ void sample_partial_kernel(const float* logits, int vocab, long long row_stride,
                                      const float* __restrict__ params,
                                      const unsigned long long* __restrict__ seeds,
                                      Best* __restrict__ partial, int blocks_per_row,
                                      unsigned long long* __restrict__ hist) {
    __shared__ Best best_scratch[32];
    TLLM_PDL_ENTER();
    const int row = blockIdx.y, b = blockIdx.x;
    const float temperature = params[2 * row], top_p = params[2 * row + 1];
    const bool nucleus = temperature > 1.0e-6f && top_p < 1.0f;
    const bool greedy = !(temperature > 1.0e-6f) || nucleus;
    if (nucleus && hist != nullptr) {
        unsigned long long* mine = hist + (size_t)row * kNucleusLevels * kNucleusBins;
        for (int i = b * blockDim.x + threadIdx.x; i < kNucleusLevels * kNucleusBins; i += blocks_per_row * blockDim.x)
            mine[i] = 0ull;
    }
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

// Picks among the blocks' candidates: of the rows with top_p < 1 if `nucleus_rows`, of the
// others if not.
__global__ void sample_final_kernel(const Best* partial, int blocks_per_row,
                                    const float* __restrict__ params, int* __restrict__ out,
                                    int nucleus_rows) {
    __shared__ Best best_scratch[32];
    TLLM_PDL_ENTER();
    const int row = blockIdx.x;
    const float temperature = params[2 * row], top_p = params[2 * row + 1];
    if ((temperature > 1.0e-6f && top_p < 1.0f) != (nucleus_rows != 0)) return;
    Best local{-FLT_MAX, INT32_MAX};
    for (int b = threadIdx.x; b < blocks_per_row; b += blockDim.x)
        local = better(local, partial[(size_t)row * blocks_per_row + b]);
    local = block_best(local, best_scratch);
    if (threadIdx.x == 0) out[row] = local.token;
}

// What the levels of the selection have settled for a row: the bin each chose and the mass
// that bin still had to give, and the row's largest logit.
struct NucleusRow {
    unsigned long long bin[kNucleusLevels], remaining[kNucleusLevels];
    float max_logit;
    int unused;
};

// The selection with a row's vocabulary shared by `blocks_per_row` blocks, as four launches
// (level 0 to 3) after sample_partial_kernel.  Level k < 3 adds the mass of the block's
// tokens whose keys agree with the bins chosen so far into hist[row][k] (in shared memory
// first, then one 64-bit integer add per bin that is not empty).  Before that, every block
// of level k > 0 finds level k-1's bin for itself from hist[row][k-1]; block 0 records it in
// settled[row] for the later levels.  Level 3 knows the whole key of the last kept token
// and leaves the block's best Gumbel score among the kept tokens in `partial`.
__global__ void nucleus_pass_kernel(const float* logits, int vocab, long long row_stride,
                                    const float* __restrict__ params,
                                    const unsigned long long* __restrict__ seeds,
                                    Best* partial, int blocks_per_row,
                                    unsigned long long* hist, NucleusRow* settled, int level) {
    __shared__ Best best_scratch[32];
    __shared__ unsigned long long bins[kNucleusBins];
    __shared__ unsigned long long scan[36];
    TLLM_PDL_ENTER();
    const int row = blockIdx.y, b = blockIdx.x;
    const float temperature = params[2 * row], top_p = params[2 * row + 1];
    if (!(temperature > 1.0e-6f && top_p < 1.0f)) return;
    const float* lg = logits + (size_t)row * row_stride;
    unsigned long long* row_hist = hist + (size_t)row * kNucleusLevels * kNucleusBins;
    NucleusRow& mine = settled[row];
    const float inv_t = 1.0f / temperature;
    const int chunk = (vocab + blocks_per_row - 1) / blocks_per_row;
    const int v0 = b * chunk, v1 = min(vocab, v0 + chunk);

    float max_logit;
    if (level == 0) {                                // the blocks' largest logits are in `partial`
        Best local{-FLT_MAX, INT32_MAX};
        for (int i = threadIdx.x; i < blocks_per_row; i += blockDim.x)
            local = better(local, partial[(size_t)row * blocks_per_row + i]);
        max_logit = block_best(local, best_scratch).value;
        if (b == 0 && threadIdx.x == 0) mine.max_logit = max_logit;
    } else {
        max_logit = mine.max_logit;
    }

    unsigned long long prefix = 0;
    for (int k = 0; k + 1 < level; ++k) prefix = (prefix << kNucleusBits) | mine.bin[k];
    if (level > 0) {                                  // settle level - 1
        const int k = level - 1;
        for (int i = threadIdx.x; i < kNucleusBins; i += blockDim.x) bins[i] = row_hist[k * kNucleusBins + i];
        if (threadIdx.x == 0) {
            scan[33] = kNucleusBins - 1;
            scan[34] = 0ull;
        }
        __syncthreads();
        unsigned long long before, own;
        const unsigned long long total = nucleus_scan(bins, scan, before, own);
        unsigned long long target;
        if (k == 0) {
            target = (unsigned long long)((double)top_p * (double)total);
            if (target < 1ull) target = 1ull;
            if (target > total) target = total;
        } else {
            target = mine.remaining[k - 1];
        }
        if (before < target && target <= before + own) {
            const int per = kNucleusBins / blockDim.x;
            int bin = threadIdx.x * per;
            unsigned long long run = before;
            while (run + bins[bin] < target) run += bins[bin++];
            scan[33] = (unsigned long long)bin;
            scan[34] = target - run;
        }
        __syncthreads();
        prefix = (prefix << kNucleusBits) | scan[33];
        if (b == 0 && threadIdx.x == 0) {
            mine.bin[k] = scan[33];
            mine.remaining[k] = scan[34];
        }
        __syncthreads();
    }

    if (level < kNucleusLevels) {
        const int shift = kNucleusBits * (kNucleusLevels - 1 - level);
        for (int i = threadIdx.x; i < kNucleusBins; i += blockDim.x) bins[i] = 0ull;
        __syncthreads();
        for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
            const float t = (max_logit - lg[v]) * inv_t;
            const unsigned long long key = nucleus_key(t);
            if (level == 0 || (key >> (shift + kNucleusBits)) == prefix) {
                const unsigned long long m = nucleus_mass(t);
                if (m) atomicAdd(&bins[(key >> shift) & (kNucleusBins - 1)], m);
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < kNucleusBins; i += blockDim.x)
            if (bins[i]) atomicAdd(&row_hist[level * kNucleusBins + i], bins[i]);
        return;
    }
    const uint64_t seed = seeds[row];
    Best local{-FLT_MAX, INT32_MAX};
    for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
        if (nucleus_key((max_logit - lg[v]) * inv_t) <= prefix) {
            const float g = -logf(-logf(uniform_of(seed, v)));
            local = better(local, Best{lg[v] + temperature * g, v});
        }
    }
    local = block_best(local, best_scratch);
    if (threadIdx.x == 0) partial[(size_t)row * blocks_per_row + b] = local;
}

// One block per row.  params[row] = {temperature, top_p}; seeds[row] is the 64-bit key.
// With `only_nucleus` rows that are greedy or have top_p == 1 are skipped (the two-stage
// kernels above have done them).
__global__ void sample_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                              const float* __restrict__ params,
                              const unsigned long long* __restrict__ seeds, int* __restrict__ out,
                              int only_nucleus) {
    __shared__ Best best_scratch[32];
    __shared__ unsigned long long hist[kNucleusBins];
    __shared__ unsigned long long scan[36];
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
        const unsigned long long last = nucleus_last_key(lg, vocab, max_logit, inv_t, top_p, hist, scan);
        local = Best{-FLT_MAX, INT32_MAX};
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
            if (nucleus_key((max_logit - lg[v]) * inv_t) <= last) {
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

// Scratch that rows with top_p < 1 need in the split form: per row three histograms of
// 2048 64-bit bins, and behind all of them one record per row.
extern "C" long long tllm_sample_nucleus_scratch_bytes(int rows) {
    return (long long)rows * (kNucleusLevels * kNucleusBins * 8 + (long long)sizeof(NucleusRow));
}

// The same result with the vocabulary of a row shared by `blocks_per_row` blocks.
// `partial` is scratch of rows * blocks_per_row * 8 bytes.  `nucleus_scratch` is null when
// no row has temperature > 1e-6 and top_p < 1, else tllm_sample_nucleus_scratch_bytes(rows)
// bytes, 8-byte aligned.
extern "C" int tllm_sample_split(const float* logits, int rows, int vocab, long long row_stride,
                                 const float* params, const unsigned long long* seeds, int* out,
                                 void* partial, int blocks_per_row, void* nucleus_scratch,
                                 cudaStream_t stream) {
    TLLM_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes");
    TLLM_REQUIRE(partial != nullptr && blocks_per_row >= 1 && blocks_per_row <= 1024 && rows <= 65535,
                 "sample: bad split");
    TLLM_REQUIRE(((uintptr_t)nucleus_scratch & 7) == 0, "sample: nucleus scratch must be 8-byte aligned");
    if (rows == 0) return 0;
    unsigned long long* hist = (unsigned long long*)nucleus_scratch;
    launch_pdl(kPdlOther, sample_partial_kernel, dim3(blocks_per_row, rows), dim3(256), 0, stream,
        logits, vocab, row_stride, params, seeds, (Best*)partial, blocks_per_row, hist);
    int rc = finish_launch("sample_partial");
    if (rc) return rc;
    launch_pdl(kPdlOther, sample_final_kernel, dim3(rows), dim3(64), 0, stream, (const Best*)partial,
               blocks_per_row, params, out, 0);
    rc = finish_launch("sample_final");
    if (rc || hist == nullptr) return rc;
    NucleusRow* settled = (NucleusRow*)(hist + (size_t)rows * kNucleusLevels * kNucleusBins);
    for (int level = 0; level <= kNucleusLevels; ++level) {
        launch_pdl(kPdlOther, nucleus_pass_kernel, dim3(blocks_per_row, rows), dim3(256), 0, stream,
            logits, vocab, row_stride, params, seeds, (Best*)partial, blocks_per_row, hist, settled, level);
        rc = finish_launch("nucleus_pass");
        if (rc) return rc;
    }
    launch_pdl(kPdlOther, sample_final_kernel, dim3(rows), dim3(64), 0, stream, (const Best*)partial,
               blocks_per_row, params, out, 1);
    return finish_launch("sample_final");
}

// The generator, for host-side restatements in tests.
extern "C" float tllm_uniform_of(unsigned long long seed, int token) { return uniform_of(seed, token); }
