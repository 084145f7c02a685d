// Per-head RMSNorm of queries and keys, rotary position encoding and the write of keys
// and values into the paged cache, in one pass over the fused q|k|v projection.
//
// The reference runs these as four launches per layer: head norm of q and of k
// (model/src/qwen3_paged_batch.cpp:160-177 through rmsnorm_kernel_cuda.cu:8-39), the
// rotate-half rotation with angle pos * theta^(-2i/hd) (rope_kernel_cuda.cu:228-261,
// table built at :186-198) and the scatter into the cache (paged_attention_cuda.cu:48-68).
// Here one warp owns one head of one token: it reads the head once, and what it
// writes is the rotated query (to `q_out`) or the rotated key / the value (to their
// page).  Norm sum, angle, sine, cosine and the rotation are float32.
//
// Cache layout of one layer: [page][0 = keys, 1 = values][kv head][slot in page][head_dim].
#include "common.cuh"

namespace tllm {

constexpr int kFlagNorm = 1;   // RMSNorm q and k heads with q_gain / k_gain
constexpr int kFlagRope = 2;   // rotate q and k
constexpr int kFlagStore = 4;  // write k and v into the cache
constexpr int kFlagQOut = 8;   // write q to q_out
constexpr int kFlagKvOut = 16; // write the processed k and v back into qkv (in place)

constexpr int kMaxHeadDim = 512;

template <typename T, typename TG>
__global__ void qk_norm_rope_store_kernel(
    T* qkv, const TG* __restrict__ q_gain, const TG* __restrict__ k_gain, float eps,
    const float* __restrict__ inv_freq, int rotary_dim, const int* __restrict__ positions,
    const int* __restrict__ token_slot, const int* __restrict__ block_table, int max_pages,
    T* __restrict__ cache, int page_size, T* __restrict__ q_out, int tokens, int q_heads,
    int kv_heads, int head_dim, int flags) {
    extern __shared__ float smem[];  // one head vector per warp
    TLLM_PDL_ENTER();
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = q_heads + 2 * kv_heads;
    const long long unit = (long long)blockIdx.x * warps_per_block + warp;
    if (unit >= (long long)tokens * heads_total) return;
    const int t = (int)(unit / heads_total);
    const int head = (int)(unit - (long long)t * heads_total);
    const int slot = token_slot[t];
    if (slot < 0) return;  // padding row
    const int pos = positions[t];

    T* src = qkv + (size_t)t * heads_total * head_dim + (size_t)head * head_dim;
    float* vec = smem + warp * head_dim;
    const bool is_q = head < q_heads;
    const bool is_k = !is_q && head < q_heads + kv_heads;

    float sumsq = 0.0f;
    for (int e = lane; e < head_dim; e += 32) {
        const float v = to_f32<T>(src[e]);
        vec[e] = v;
        sumsq += v * v;
    }
    if ((is_q || is_k) && (flags & kFlagNorm)) {
        sumsq = warp_sum(sumsq);
        const float scale = 1.0f / sqrtf(sumsq / (float)head_dim + eps);
        const TG* gain = is_q ? q_gain : k_gain;
        for (int e = lane; e < head_dim; e += 32) vec[e] = to_f32<TG>(gain[e]) * vec[e] * scale;
    }
    __syncwarp();

    T* dst = nullptr;
    if (is_q) {
        if (flags & kFlagQOut) dst = q_out + (size_t)t * q_heads * head_dim + (size_t)head * head_dim;
    } else if (flags & kFlagStore) {
        const int kvh = is_k ? head - q_heads : head - q_heads - kv_heads;
        const int page = block_table[(size_t)slot * max_pages + pos / page_size];
        if (page >= 0) {
            dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * kv_heads + kvh) * page_size +
                           (pos % page_size)) * head_dim;
        }
    }
    T* dst2 = (!is_q && (flags & kFlagKvOut)) ? src : nullptr;
    if (!dst && !dst2) return;

    const int half = rotary_dim >> 1;
    const bool rotate = (is_q || is_k) && (flags & kFlagRope) && half > 0;
    for (int e = lane; e < head_dim; e += 32) {
        float v = vec[e];
        if (rotate && e < rotary_dim) {
            // pair (i, i + half): x'_i = x_i cos a - x_{i+half} sin a; x'_{i+half} = x_i sin a + x_{i+half} cos a
            const int i = e < half ? e : e - half;
            float s, c;
            sincosf((float)pos * inv_freq[i], &s, &c);
            v = e < half ? vec[e] * c - vec[e + half] * s : vec[e - half] * s + vec[e] * c;
        }
        if (dst) dst[e] = from_f32<T>(v);
        if (dst2) dst2[e] = from_f32<T>(v);
    }
}

// Vector form for head widths 64, 128 and 256 with the whole head rotated: one block per
// token.  The block first writes the token's cosines and sines to shared memory (once, not
// once per head), then its warps take the heads in turn.  A lane holds VEC = head_dim / 32
// neighbouring elements (one 4-, 8- or 16-byte access); the rotation partner of an element
// is VEC * 16 elements away, that is, in lane ^ 16.
template <typename T, int VEC> struct VecIO;
template <int VEC> struct VecIO<bf16, VEC> {
    // what a load leaves in registers until it is needed: half the registers of the float form
    struct Raw { uint32_t w[VEC / 2]; };
    static __device__ __forceinline__ Raw load_raw(const bf16* p) {
        Raw raw;
        if constexpr (VEC == 2) {
            raw.w[0] = *reinterpret_cast<const uint32_t*>(p);
        } else if constexpr (VEC == 4) {
            const uint2 u = *reinterpret_cast<const uint2*>(p);
            raw.w[0] = u.x; raw.w[1] = u.y;
        } else {
            const uint4 u = *reinterpret_cast<const uint4*>(p);
            raw.w[0] = u.x; raw.w[1] = u.y; raw.w[2] = u.z; raw.w[3] = u.w;
        }
        return raw;
    }
    static __device__ __forceinline__ void unpack(const Raw& raw, float (&v)[VEC]) {
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
            v[2 * i] = __uint_as_float(raw.w[i] << 16);
            v[2 * i + 1] = __uint_as_float(raw.w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[VEC]) { unpack(load_raw(p), v); }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[VEC]) {
        if constexpr (VEC == 2) {
            *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
        } else if constexpr (VEC == 4) {
            uint2 raw;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
            h[0] = __floats2bfloat162_rn(v[0], v[1]);
            h[1] = __floats2bfloat162_rn(v[2], v[3]);
            *reinterpret_cast<uint2*>(p) = raw;
        } else {
            uint4 raw;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            *reinterpret_cast<uint4*>(p) = raw;
        }
    }
};
template <int VEC> struct VecIO<float, VEC> {
    struct Raw { float v[VEC]; };
    static __device__ __forceinline__ Raw load_raw(const float* p) {
        Raw raw;
#pragma unroll
        for (int i = 0; i < VEC; i += 2) {
            const float2 f = *reinterpret_cast<const float2*>(p + i);
            raw.v[i] = f.x; raw.v[i + 1] = f.y;
        }
        return raw;
    }
    static __device__ __forceinline__ void unpack(const Raw& raw, float (&v)[VEC]) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = raw.v[i];
    }
    static __device__ __forceinline__ void load(const float* p, float (&v)[VEC]) { unpack(load_raw(p), v); }
    static __device__ __forceinline__ void store(float* p, const float (&v)[VEC]) {
#pragma unroll
        for (int i = 0; i < VEC; i += 2) *reinterpret_cast<float2*>(p + i) = make_float2(v[i], v[i + 1]);
    }
};

template <typename T, typename TG, int VEC>
__global__ void __launch_bounds__(256, (VEC <= 4 && sizeof(T) == 2) ? 4 : 2) qk_norm_rope_store_vec_kernel(
    T* qkv, const TG* __restrict__ q_gain, const TG* __restrict__ k_gain, float eps,
    const float* __restrict__ inv_freq, const int* __restrict__ positions,
    const int* __restrict__ token_slot, const int* __restrict__ block_table, int max_pages,
    T* __restrict__ cache, int page_size, T* __restrict__ q_out, int q_heads, int kv_heads, int flags) {
    constexpr int HD = VEC * 32, HALF = HD / 2;
    __shared__ float cs[HALF], sn[HALF];
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const bool rope = (flags & kFlagRope) != 0;
    const int heads_total = q_heads + 2 * kv_heads;
    const int e0 = lane * VEC;
    T* row = qkv + (size_t)t * heads_total * HD;
    // With few tokens the heads of a token are spread over gridDim.y blocks (one round per warp);
    // with many a warp takes several heads, and loads kRounds of them before it works on the
    // first, so that their latencies overlap.  The first loads are issued before the angles are
    // computed (sincosf of a large argument is slow) and before the page is looked up.
    constexpr int kRounds = 6;
    const int stride = warps * gridDim.y;
    typename VecIO<T, VEC>::Raw xs[kRounds];
    auto load_heads = [&](int first) {
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int head = first + r * stride;
            if (head < heads_total) xs[r] = VecIO<T, VEC>::load_raw(row + (size_t)head * HD + e0);
        }
    };
    load_heads(blockIdx.y * warps + warp);
    if (rope)
        for (int i = threadIdx.x; i < HALF; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
    float gq[VEC], gk[VEC];
    if (flags & kFlagNorm) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) { gq[i] = to_f32<TG>(q_gain[e0 + i]); gk[i] = to_f32<TG>(k_gain[e0 + i]); }
    }
    int page = -1;
    if (flags & kFlagStore) page = block_table[(size_t)slot * max_pages + pos / page_size];
    __syncthreads();
    for (int first = blockIdx.y * warps + warp; first < heads_total; first += stride * kRounds) {
        if (first != blockIdx.y * warps + warp) load_heads(first);
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int head = first + r * stride;
            if (head >= heads_total) break;
            float x[VEC];
            VecIO<T, VEC>::unpack(xs[r], x);
            const bool is_q = head < q_heads, is_k = !is_q && head < q_heads + kv_heads;
            T* src = row + (size_t)head * HD + e0;
            if ((is_q || is_k) && (flags & kFlagNorm)) {
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < VEC; ++i) ss += x[i] * x[i];
                ss = warp_sum(ss);
                const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
                for (int i = 0; i < VEC; ++i) x[i] = (is_q ? gq[i] : gk[i]) * x[i] * scale;
            }
            if ((is_q || is_k) && rope) {
                const bool low = lane < 16;
                const int f0 = low ? e0 : e0 - HALF;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
                    const float c = cs[f0 + i], s = sn[f0 + i];
                    x[i] = low ? x[i] * c - other * s : other * s + x[i] * c;
                }
            }
            if (is_q) {
                if (flags & kFlagQOut) VecIO<T, VEC>::store(q_out + ((size_t)t * q_heads + head) * HD + e0, x);
            } else {
                if ((flags & kFlagStore) && page >= 0) {
                    const int kvh = is_k ? head - q_heads : head - q_heads - kv_heads;
                    T* dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * kv_heads + kvh) * page_size +
                                      (pos % page_size)) * HD + e0;
                    VecIO<T, VEC>::store(dst, x);
                }
                if (flags & kFlagKvOut) VecIO<T, VEC>::store(src, x);
            }
        }
    }
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_qk_norm_rope_store(
    void* qkv, const void* q_gain, const void* k_gain, int gain_dtype, float eps,
    const float* inv_freq, int rotary_dim, const int* positions, const int* token_slot,
    const int* block_table, int max_pages, void* cache, int page_size, void* q_out, int dtype,
    int tokens, int q_heads, int kv_heads, int head_dim, int flags, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0, "qk_norm_rope_store: bad sizes");
    TLLM_REQUIRE(head_dim > 0 && head_dim <= kMaxHeadDim,
                 "qk_norm_rope_store: head_dim %d outside 1..%d", head_dim, kMaxHeadDim);
    TLLM_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                 "qk_norm_rope_store: rotary_dim %d must be even and at most head_dim %d",
                 rotary_dim, head_dim);
    TLLM_REQUIRE(!(flags & kFlagRope) || inv_freq != nullptr, "qk_norm_rope_store: rotation without frequencies");
    TLLM_REQUIRE(!(flags & kFlagNorm) || (q_gain && k_gain), "qk_norm_rope_store: norm without gains");
    TLLM_REQUIRE(!(flags & kFlagStore) || (cache && block_table && page_size > 0 && max_pages > 0),
                 "qk_norm_rope_store: store without cache");
    TLLM_REQUIRE(!(flags & kFlagQOut) || q_out, "qk_norm_rope_store: no query output");
    TLLM_REQUIRE(gain_dtype == kBF16 || gain_dtype == kF32, "qk_norm_rope_store: unknown gain dtype");
    if (tokens == 0) return 0;
    const bool whole_rotation = !(flags & kFlagRope) || rotary_dim == head_dim;
    const auto al = [](const void* p, int bytes) { return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0; };
    if (whole_rotation && (head_dim == 64 || head_dim == 128 || head_dim == 256)) {
        const int need = dtype == kBF16 ? (head_dim / 32) * 2 : 8;     // widest access of the vector form
        if (al(qkv, need) && al(cache, need) && al(q_out, need) && (dtype == kBF16 || dtype == kF32)) {
            const int vblock = 256;
            const int vgroups = tokens <= 64 ? (q_heads + 2 * kv_heads + 7) / 8 : 1;
#define VLAUNCH(T, TG, VEC)                                                                         \
    launch_pdl(kPdlQk, qk_norm_rope_store_vec_kernel<T, TG, VEC>, dim3(tokens, vgroups), dim3(vblock), 0, stream, \
        (T*)qkv, (const TG*)q_gain, (const TG*)k_gain, eps, inv_freq, positions, token_slot,        \
        block_table, max_pages, (T*)cache, page_size, (T*)q_out, q_heads, kv_heads, flags)
#define VDISPATCH(T, TG)                                              \
    do {                                                              \
        if (head_dim == 64) VLAUNCH(T, TG, 2);                        \
        else if (head_dim == 128) VLAUNCH(T, TG, 4);                  \
        else VLAUNCH(T, TG, 8);                                       \
    } while (0)
            if (dtype == kBF16) {
                if (gain_dtype == kBF16) VDISPATCH(bf16, bf16); else VDISPATCH(bf16, float);
            } else {
                if (gain_dtype == kBF16) VDISPATCH(float, bf16); else VDISPATCH(float, float);
            }
#undef VDISPATCH
#undef VLAUNCH
            return finish_launch("qk_norm_rope_store");
        }
    }
    const int warps = 4, block = warps * 32;
    const long long units = (long long)tokens * (q_heads + 2 * kv_heads);
    const int grid = (int)((units + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
#define LAUNCH(T, TG)                                                                            \
    launch_pdl(kPdlQk, qk_norm_rope_store_kernel<T, TG>, dim3(grid), dim3(block), smem, stream,          \
        (T*)qkv, (const TG*)q_gain, (const TG*)k_gain, eps, inv_freq, rotary_dim, positions,     \
        token_slot, block_table, max_pages, (T*)cache, page_size, (T*)q_out, tokens, q_heads,    \
        kv_heads, head_dim, flags)
    if (dtype == kBF16) {
        if (gain_dtype == kBF16) LAUNCH(bf16, bf16); else LAUNCH(bf16, float);
    } else if (dtype == kF32) {
        if (gain_dtype == kBF16) LAUNCH(float, bf16); else LAUNCH(float, float);
    } else {
        TLLM_REQUIRE(false, "qk_norm_rope_store: unknown dtype %d", dtype);
    }
#undef LAUNCH
    return finish_launch("qk_norm_rope_store");
}
