// Attention over the paged cache, general form: any head width up to 512, any number
// of heads and groups, both storage types, optional sliding window.  One block owns
// one (token, query head); its warps walk disjoint keys with an online softmax and are
// merged at the end.  It is the kernel of the float32 path and the fallback of the
// bfloat16 path for shapes the tensor-core kernels refuse.
//
// Same mathematics as the reference (kernels/src/paged_attention_cuda.cu:70-120):
// scores (q . k_j) / sqrt(hd) for the keys j <= pos of the token's own request, softmax
// with the maximum subtracted, weighted sum of values, all float32; the causal mask is
// the bound j <= pos, so later tokens of the same step, already in the cache, are never
// read.  Unlike the reference no score ever goes to global memory.
//
// The order of the additions for a (request, position, head) depends only on the
// position and the window, never on what else is in the batch or on the pages used.
#include "common.cuh"

namespace tllm {

constexpr int kWarps = 4;

template <typename T, int CHUNKS>
__global__ void paged_attention_general_kernel(
    const T* q, const T* cache, const int* __restrict__ positions,
    const int* __restrict__ token_slot, const int* __restrict__ block_table, int max_pages,
    int page_size, int q_heads, int kv_heads, int head_dim, int window, float scale,
    T* __restrict__ out) {
    extern __shared__ float smem[];
    TLLM_PDL_ENTER();
    float* qs = smem;                          // [head_dim]
    float* acc_s = smem + head_dim;            // [kWarps][head_dim]
    float* m_s = acc_s + kWarps * head_dim;    // [kWarps]
    float* l_s = m_s + kWarps;                 // [kWarps]

    const int head = blockIdx.x, t = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* dst = out + ((size_t)t * q_heads + head) * head_dim;
    const int slot = token_slot[t];
    if (slot < 0) {
        for (int e = threadIdx.x; e < head_dim; e += blockDim.x) dst[e] = from_f32<T>(0.0f);
        return;
    }
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int g = head / (q_heads / kv_heads);
    const T* qsrc = q + ((size_t)t * q_heads + head) * head_dim;
    for (int e = threadIdx.x; e < head_dim; e += blockDim.x) qs[e] = to_f32<T>(qsrc[e]) * scale;
    __syncthreads();

    const int* table = block_table + (size_t)slot * max_pages;
    float m = -INFINITY, l = 0.0f;
    float acc[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) acc[c] = 0.0f;

    for (int j = lo + warp; j <= pos; j += kWarps) {
        const int page = table[j / page_size];
        if (page < 0) continue;  // a page the window has passed; never inside [lo, pos]
        const size_t base = (((size_t)page * 2) * kv_heads + g) * page_size + (j % page_size);
        const T* kp = cache + base * head_dim;
        const T* vp = cache + (base + (size_t)kv_heads * page_size) * head_dim;
        float dot = 0.0f;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int e = lane + 32 * c;
            if (e < head_dim) dot += qs[e] * to_f32<T>(kp[e]);
        }
        dot = warp_sum(dot);
        const float m_new = fmaxf(m, dot);
        const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first key
        const float p = expf(dot - m_new);
        l = l * corr + p;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int e = lane + 32 * c;
            if (e < head_dim) acc[c] = acc[c] * corr + p * to_f32<T>(vp[e]);
        }
        m = m_new;
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int e = lane + 32 * c;
        if (e < head_dim) acc_s[warp * head_dim + e] = acc[c];
    }
    __syncthreads();
    float mm = m_s[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) mm = fmaxf(mm, m_s[w]);
    float w_scale[kWarps], total = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        w_scale[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - mm);
        total += l_s[w] * w_scale[w];
    }
    const float inv = 1.0f / total;
    for (int e = threadIdx.x; e < head_dim; e += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += acc_s[w * head_dim + e] * w_scale[w];
        dst[e] = from_f32<T>(v * inv);
    }
}

template <typename T>
static int launch_general(const void* q, const void* cache, const int* positions,
                          const int* token_slot, const int* block_table, int max_pages,
                          int page_size, int tokens, int q_heads, int kv_heads, int head_dim,
                          int window, float scale, void* out, cudaStream_t stream) {
    const dim3 grid(q_heads, tokens), block(kWarps * 32);
    const size_t smem = ((size_t)head_dim * (1 + kWarps) + 2 * kWarps) * sizeof(float);
    const int chunks = (head_dim + 31) / 32;
#define LAUNCH(C)                                                                              \
    launch_pdl(kPdlAttention, paged_attention_general_kernel<T, C>, grid, block, smem, stream,                 \
        (const T*)q, (const T*)cache, positions, token_slot, block_table, max_pages, page_size, \
        q_heads, kv_heads, head_dim, window, scale, (T*)out)
    if (chunks <= 1) LAUNCH(1);
    else if (chunks <= 2) LAUNCH(2);
    else if (chunks <= 4) LAUNCH(4);
    else if (chunks <= 8) LAUNCH(8);
    else LAUNCH(16);
#undef LAUNCH
    return finish_launch("paged_attention_general");
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_paged_attention_general(
    const void* q, const void* cache, const int* positions, const int* token_slot,
    const int* block_table, int max_pages, int page_size, int dtype, int tokens, int q_heads,
    int kv_heads, int head_dim, int window, float scale, void* out, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
                 "paged_attention: %d query heads over %d key/value heads", q_heads, kv_heads);
    TLLM_REQUIRE(head_dim > 0 && head_dim <= 512, "paged_attention: head_dim %d outside 1..512", head_dim);
    TLLM_REQUIRE(page_size > 0 && max_pages > 0, "paged_attention: bad page geometry");
    TLLM_REQUIRE(tokens <= 65535, "paged_attention: %d tokens in one step exceed 65535", tokens);
    if (tokens == 0) return 0;
    if (dtype == kBF16)
        return launch_general<bf16>(q, cache, positions, token_slot, block_table, max_pages, page_size,
                                    tokens, q_heads, kv_heads, head_dim, window, scale, out, stream);
    if (dtype == kF32)
        return launch_general<float>(q, cache, positions, token_slot, block_table, max_pages, page_size,
                                     tokens, q_heads, kv_heads, head_dim, window, scale, out, stream);
    TLLM_REQUIRE(false, "paged_attention: unknown dtype %d", dtype);
}
