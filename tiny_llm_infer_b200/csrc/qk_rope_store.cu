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
// once per head), then its warps take the heads in turn.  A lane holds eight neighbouring
// elements of a head (one 16-byte access in bfloat16), so a head is HD / 8 lanes and a warp
// works on 32 / (HD / 8) heads at once; the rotation partner of an element is HD / 2 elements
// away, that is, HD / 16 lanes.  With many tokens the kernel is bound by the instructions it
// issues, not by memory (one head per warp and four elements per lane: 158 warp instructions
// per head, 2 TB/s at 2048 tokens of Qwen3-8B sizes), hence the wide lanes, the cosines and signed
// sines kept in registers for all heads of the token, and the three rounds of heads loaded before
// the first is worked on.
template <typename T> struct HeadVec8;
template <> struct HeadVec8<bf16> {
    struct Raw { uint4 u; };
    static __device__ __forceinline__ Raw load_raw(const bf16* p) { return Raw{*reinterpret_cast<const uint4*>(p)}; }
    static __device__ __forceinline__ void unpack(const Raw& raw, float (&v)[8]) {
        const uint32_t w[4] = {raw.u.x, raw.u.y, raw.u.z, raw.u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
    static __device__ __forceinline__ float inv_root(float x) { return rsqrtf(x); }
};
template <> struct HeadVec8<float> {
    struct Raw { float4 a, b; };
    static __device__ __forceinline__ Raw load_raw(const float* p) {
        return Raw{*reinterpret_cast<const float4*>(p), *reinterpret_cast<const float4*>(p + 4)};
    }
    static __device__ __forceinline__ void unpack(const Raw& raw, float (&v)[8]) {
        v[0] = raw.a.x; v[1] = raw.a.y; v[2] = raw.a.z; v[3] = raw.a.w;
        v[4] = raw.b.x; v[5] = raw.b.y; v[6] = raw.b.z; v[7] = raw.b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    static __device__ __forceinline__ float inv_root(float x) { return 1.0f / sqrtf(x); }   // the 32-bit path: exact root and quotient
};

// TABLE: the cosines and sines of the step's tokens come from `rope_table` ([tokens][2][HD / 2]
// float32, made once per step by rope_table_kernel and shared by all layers) instead of being
// computed here, which takes 64 sincosf, the shared memory and the barrier out of every block.
// ROUNDS: how many heads a warp loads before it works on the first.  With many tokens a block of four
// warps with six loads each in flight keeps more bytes on their way per SM than eight warps with three
// (the kernel is bound by the latency of its loads, not by its instructions).
template <typename T, typename TG, int HD, bool TABLE, int ROUNDS>
__global__ void __launch_bounds__(256) qk_norm_rope_store_vec_kernel(
    T* qkv, const TG* __restrict__ q_gain, const TG* __restrict__ k_gain, float eps,
    const float* __restrict__ inv_freq, const float* rope_table, const int* __restrict__ positions,
    const int* __restrict__ token_slot, const int* __restrict__ block_table, int max_pages,
    T* __restrict__ cache, int page_size, T* __restrict__ q_out, int q_heads, int kv_heads, int flags) {
    constexpr int HALF = HD / 2, LPH = HD / 8, HPW = 32 / LPH;   // lanes per head, heads per warp
    __shared__ __align__(16) float cs[HALF], sn[HALF];
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int sub = lane / LPH, l = lane % LPH;
    const bool rope = (flags & kFlagRope) != 0, norm = (flags & kFlagNorm) != 0;
    const int heads_total = q_heads + 2 * kv_heads;
    const int e0 = l * 8;
    T* row = qkv + (size_t)t * heads_total * HD;
    // With few tokens the heads of a token are spread over gridDim.y blocks (one round per warp);
    // with many a warp takes several rounds of heads, and loads kRounds of them before it works on
    // the first, so that their latencies overlap.  The first loads are issued before the angles
    // are computed and before the page is looked up.
    constexpr int kRounds = ROUNDS;
    const int stride = warps * HPW * gridDim.y;
    const int head0 = (blockIdx.y * warps + warp) * HPW + sub;
    typename HeadVec8<T>::Raw xs[kRounds];
    auto load_heads = [&](int first) {
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int head = first + r * stride;
            if (head < heads_total) xs[r] = HeadVec8<T>::load_raw(row + (size_t)head * HD + e0);
        }
    };
    load_heads(head0);
    const bool low = l < LPH / 2;
    float4 tc0, tc1, ts0, ts1;                        // TABLE: this lane's eight cosines and sines, on their way
    if constexpr (TABLE) {
        if (rope) {
            const float* row_c = rope_table + (size_t)t * HD + (low ? e0 : e0 - HALF);
            tc0 = *reinterpret_cast<const float4*>(row_c);
            tc1 = *reinterpret_cast<const float4*>(row_c + 4);
            ts0 = *reinterpret_cast<const float4*>(row_c + HALF);
            ts1 = *reinterpret_cast<const float4*>(row_c + HALF + 4);
        }
    } else {
        if (rope)
            for (int i = threadIdx.x; i < HALF; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
    }
    float gq[8], gk[8];
    if (norm) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { gq[i] = to_f32<TG>(q_gain[e0 + i]); gk[i] = to_f32<TG>(k_gain[e0 + i]); }
    }
    int page = -1;
    if (flags & kFlagStore) page = block_table[(size_t)slot * max_pages + pos / page_size];
    if constexpr (!TABLE) __syncthreads();
    // pair (i, i + HALF): x'_i = x_i cos a - x_{i+HALF} sin a; x'_{i+HALF} = x_i sin a + x_{i+HALF} cos a,
    // for both halves x' = x cos a + partner * (-+ sin a): cosines and signed sines of this lane's elements
    float cc[8], sx[8];
    if (rope) {
        const int f0 = low ? e0 : e0 - HALF;
        float4 c0, c1, s0, s1;
        if constexpr (TABLE) {
            c0 = tc0; c1 = tc1; s0 = ts0; s1 = ts1;
        } else {
            c0 = *reinterpret_cast<const float4*>(cs + f0); c1 = *reinterpret_cast<const float4*>(cs + f0 + 4);
            s0 = *reinterpret_cast<const float4*>(sn + f0); s1 = *reinterpret_cast<const float4*>(sn + f0 + 4);
        }
        cc[0] = c0.x; cc[1] = c0.y; cc[2] = c0.z; cc[3] = c0.w; cc[4] = c1.x; cc[5] = c1.y; cc[6] = c1.z; cc[7] = c1.w;
        sx[0] = s0.x; sx[1] = s0.y; sx[2] = s0.z; sx[3] = s0.w; sx[4] = s1.x; sx[5] = s1.y; sx[6] = s1.z; sx[7] = s1.w;
        if (low) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sx[i] = -sx[i];
        }
    }
    for (int first = head0; first < heads_total; first += stride * kRounds) {
        if (first != head0) load_heads(first);
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int head = first + r * stride;
            // heads of one warp differ by less than HPW: whether a head exists may differ inside the
            // warp, so lanes without one keep going (with a copy of a head that exists) for the shuffles
            const bool live = head < heads_total;
            if (__all_sync(0xffffffffu, !live)) break;
            float x[8];
            HeadVec8<T>::unpack(xs[r], x);
            const bool is_q = head < q_heads, is_k = !is_q && head < q_heads + kv_heads;
            if (norm) {
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
                for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (is_q || is_k) {
                    const float scale = HeadVec8<T>::inv_root(ss / (float)HD + eps);
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = (is_q ? gq[i] : gk[i]) * x[i] * scale;
                }
            }
            if (rope) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float other = __shfl_xor_sync(0xffffffffu, x[i], LPH / 2);
                    if (is_q || is_k) x[i] = fmaf(x[i], cc[i], other * sx[i]);
                }
            }
            if (!live) continue;
            if (is_q) {
                if (flags & kFlagQOut) HeadVec8<T>::store(q_out + ((size_t)t * q_heads + head) * HD + e0, x);
            } else {
                if ((flags & kFlagStore) && page >= 0) {
                    const int kvh = is_k ? head - q_heads : head - q_heads - kv_heads;
                    T* dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * kv_heads + kvh) * page_size +
                                      (pos % page_size)) * HD + e0;
                    HeadVec8<T>::store(dst, x);
                }
                if (flags & kFlagKvOut) HeadVec8<T>::store(row + (size_t)head * HD + e0, x);
            }
        }
    }
}

// table[t][0][i] = cos(pos_t * inv_freq[i]), table[t][1][i] = sin(pos_t * inv_freq[i]), i < half: the
// angle is the float32 product, as in the kernels above that compute it themselves.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int half,
                                  int tokens, float* __restrict__ table) {
    TLLM_PDL_ENTER();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * half) return;
    const int t = idx / half, i = idx - t * half;
    float s, c;
    sincosf((float)positions[t] * inv_freq[i], &s, &c);
    table[(size_t)t * 2 * half + i] = c;
    table[(size_t)t * 2 * half + half + i] = s;
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_rope_table(const int* positions, const float* inv_freq, int half, int tokens, float* table,
                               cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && half > 0 && positions && inv_freq && table, "rope_table: bad arguments");
    if (tokens == 0) return 0;
    const long long n = (long long)tokens * half;
    launch_pdl(kPdlOther, rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, positions, inv_freq,
               half, tokens, table);
    return finish_launch("rope_table");
}

// rope_table: optional, [tokens][2][head_dim / 2] float32 from tllm_rope_table for the same positions and
// frequencies (used by the vector form when the whole head is rotated; ignored otherwise).
extern "C" int tllm_qk_norm_rope_store(
    void* qkv, const void* q_gain, const void* k_gain, int gain_dtype, float eps,
    const float* inv_freq, int rotary_dim, const int* positions, const int* token_slot,
    const int* block_table, int max_pages, void* cache, int page_size, void* q_out, int dtype,
    int tokens, int q_heads, int kv_heads, int head_dim, int flags, const float* rope_table, cudaStream_t stream) {
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
        const int need = 16;                                           // widest access of the vector form
        if (al(qkv, need) && al(cache, need) && al(q_out, need) && (dtype == kBF16 || dtype == kF32)) {
            const int vblock = 256;
            const int per_block = 8 * (32 / (head_dim / 8));           // heads a block takes in one round
            const int vgroups = tokens <= 64 ? (q_heads + 2 * kv_heads + per_block - 1) / per_block : 1;
            const bool table = rope_table != nullptr && (flags & kFlagRope) && al(rope_table, 16);
            const bool deep = tokens > 64;                                  // see ROUNDS above
#define VLAUNCH1(T, TG, HD, TAB, ROUNDS, BLOCK)                                                     \
    launch_pdl(kPdlQk, qk_norm_rope_store_vec_kernel<T, TG, HD, TAB, ROUNDS>, dim3(tokens, vgroups), dim3(BLOCK), 0, stream, \
        (T*)qkv, (const TG*)q_gain, (const TG*)k_gain, eps, inv_freq, rope_table, positions, token_slot, \
        block_table, max_pages, (T*)cache, page_size, (T*)q_out, q_heads, kv_heads, flags)
#define VLAUNCH(T, TG, HD)                                                                          \
    do {                                                                                            \
        if (table && deep) VLAUNCH1(T, TG, HD, true, 6, 128);                                       \
        else if (table) VLAUNCH1(T, TG, HD, true, 3, vblock);                                       \
        else if (deep) VLAUNCH1(T, TG, HD, false, 6, 128);                                          \
        else VLAUNCH1(T, TG, HD, false, 3, vblock);                                                 \
    } while (0)
#define VDISPATCH(T, TG)                                              \
    do {                                                              \
        if (head_dim == 64) VLAUNCH(T, TG, 64);                       \
        else if (head_dim == 128) VLAUNCH(T, TG, 128);                \
        else VLAUNCH(T, TG, 256);                                     \
    } while (0)
            if (dtype == kBF16) {
                if (gain_dtype == kBF16) VDISPATCH(bf16, bf16); else VDISPATCH(bf16, float);
            } else {
                if (gain_dtype == kBF16) VDISPATCH(float, bf16); else VDISPATCH(float, float);
            }
#undef VDISPATCH
#undef VLAUNCH
#undef VLAUNCH1
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
