// Attention of prompt portions over the paged cache, bfloat16, flash-attention style on
// mma.sync tensor-core tiles.
//
// The reference treats every prompt token as a decode query of its own and re-reads all
// earlier keys and values for it, with the scores round-tripping through global memory
// (kernels/src/paged_attention_cuda.cu:70-120).  Here a block owns 64 consecutive query
// rows of one portion and one query head: it walks the request's keys in tiles of 64,
// taken from the pages (the portion's own keys were written to the cache just before),
// keeps S = Q K^T and the online softmax in float32 registers and accumulates P V in
// float32.  The causal rule is per row, key <= position of the row (and, with a window,
// key > position - window); tiles that no row of a warp may see are skipped by that warp.
// Keys and values are staged by cp.async in two buffers so that the next tile loads while
// this one is multiplied.
//
// Takes head widths 64 and 128 and page sizes that are multiples of 16; the caller sends
// other shapes to the general kernel.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace tllm {

constexpr int kPfWarps = 4;
constexpr int kBM = 64;   // query rows per block
constexpr int kBN = 64;   // keys per tile

template <int HD>
__global__ void __launch_bounds__(kPfWarps * 32)
paged_attention_prefill_kernel(const bf16* q, const bf16* cache,
                               const int* __restrict__ seg_info, const int* __restrict__ tiles,
                               const int* __restrict__ block_table, int max_pages, int page_size,
                               int q_heads, int kv_heads, int window, float scale_log2e,
                               bf16* __restrict__ out) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    TLLM_PDL_ENTER();
    constexpr int kChunks = HD / 8;
    constexpr int kTileBytes = kBN * HD * 2;
    const int seg = tiles[2 * blockIdx.x], q_off = tiles[2 * blockIdx.x + 1];
    const int head = blockIdx.y;
    const int slot = seg_info[4 * seg], start = seg_info[4 * seg + 1];
    const int len = seg_info[4 * seg + 2], pos0 = seg_info[4 * seg + 3];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = head / (q_heads / kv_heads);
    const int* table = block_table + (size_t)slot * max_pages;

    const int rows_here = min(kBM, len - q_off);
    const int first_pos = pos0 + q_off, last_pos = first_pos + rows_here - 1;
    const int lo_all = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int kt_first = lo_all / kBN, kt_last = last_pos / kBN;

    // ---- this warp's 16 query rows as A fragments
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;         // row within the block
    const bool v_lo = r_lo < rows_here, v_hi = r_hi < rows_here;
    const int p_lo = first_pos + r_lo, p_hi = first_pos + r_hi;        // their positions
    const bf16* q_lo = q + ((size_t)(start + q_off + r_lo) * q_heads + head) * HD;
    const bf16* q_hi = q + ((size_t)(start + q_off + r_hi) * q_heads + head) * HD;
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const int c0 = ks * 16 + (lane & 3) * 2;
        qa[ks][0] = v_lo ? *reinterpret_cast<const uint32_t*>(q_lo + c0) : 0u;
        qa[ks][1] = v_hi ? *reinterpret_cast<const uint32_t*>(q_hi + c0) : 0u;
        qa[ks][2] = v_lo ? *reinterpret_cast<const uint32_t*>(q_lo + c0 + 8) : 0u;
        qa[ks][3] = v_hi ? *reinterpret_cast<const uint32_t*>(q_hi + c0 + 8) : 0u;
    }
    // positions this warp's rows span (for skipping whole tiles)
    const int w_first = first_pos + warp * 16;
    const int w_last = min(w_first + 15, last_pos);
    const int w_lo = (window > 0 && w_first - window + 1 > 0) ? w_first - window + 1 : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    auto issue = [&](int kt, int stage) {
        const uint32_t ks = smem_u32(smem_raw + (size_t)stage * 2 * kTileBytes);
        const uint32_t vs = ks + kTileBytes;
#pragma unroll
        for (int i = 0; i < (kBN * kChunks) / (kPfWarps * 32); ++i) {
            const int c = threadIdx.x + kPfWarps * 32 * i, row = c / kChunks, chunk = c % kChunks;
            const int key = kt * kBN + row;
            const int page = key <= last_pos ? table[key / page_size] : -1;
            const bool ok = page >= 0;
            const size_t off = ((size_t)(ok ? page : 0) * 2 * kv_heads + g) * page_size + (key % page_size);
            cp_async_16(ks + swizzled<HD>(row, chunk), cache + off * HD + chunk * 8, ok);
            cp_async_16(vs + swizzled<HD>(row, chunk),
                        cache + (off + (size_t)kv_heads * page_size) * HD + chunk * 8, ok);
        }
        cp_async_commit();
    };

    issue(kt_first, 0);
    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int stage = (kt - kt_first) & 1;
        if (kt + 1 <= kt_last) {
            issue(kt + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key0 = kt * kBN;
        const bool active = warp * 16 < rows_here && key0 <= w_last && key0 + kBN - 1 >= w_lo;
        if (active) {
            const uint32_t ks_base = smem_u32(smem_raw + (size_t)stage * 2 * kTileBytes);
            const uint32_t vs_base = ks_base + kTileBytes;
            const int mid = lane >> 3, mrow = lane & 7;
            float s[kBN / 8][4];
#pragma unroll
            for (int i = 0; i < kBN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int nt2 = 0; nt2 < kBN / 16; ++nt2) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, ks_base + swizzled<HD>(nt2 * 16 + (mid >> 1) * 8 + mrow, 2 * ks + (mid & 1)));
                    const uint32_t b0[2] = {kb[0], kb[1]}, b1[2] = {kb[2], kb[3]};
                    mma_bf16_16816(s[2 * nt2], qa[ks], b0);
                    mma_bf16_16816(s[2 * nt2 + 1], qa[ks], b1);
                }
            }
            const int key_base = key0 + (lane & 3) * 2;
            const int min_lo = window > 0 ? p_lo - window + 1 : 0, min_hi = window > 0 ? p_hi - window + 1 : 0;
            float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < kBN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = key_base + nt * 8 + e;
                    s[nt][e] = (j <= p_lo && j >= min_lo) ? s[nt][e] * scale_log2e : -INFINITY;
                    s[nt][2 + e] = (j <= p_hi && j >= min_hi) ? s[nt][2 + e] * scale_log2e : -INFINITY;
                    tmax_lo = fmaxf(tmax_lo, s[nt][e]);
                    tmax_hi = fmaxf(tmax_hi, s[nt][2 + e]);
                }
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
            const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
            const float ms_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
            const float c_lo = exp2f(m_lo - ms_lo), c_hi = exp2f(m_hi - ms_hi);
            m_lo = mn_lo;
            m_hi = mn_hi;
            float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int nt = 0; nt < kBN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[nt][e] = exp2f(s[nt][e] - ms_lo);
                    s[nt][2 + e] = exp2f(s[nt][2 + e] - ms_hi);
                    sum_lo += s[nt][e];
                    sum_hi += s[nt][2 + e];
                }
            l_lo = l_lo * c_lo + sum_lo;
            l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
            }
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk) {
                const uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                        pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                                        pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int c = 0; c < HD / 8; c += 2) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vs_base + swizzled<HD>(kk * 16 + (mid & 1) * 8 + mrow, c + (mid >> 1)));
                    const uint32_t b0[2] = {vb[0], vb[1]}, b1[2] = {vb[2], vb[3]};
                    mma_bf16_16816(o[c], pa, b0);
                    mma_bf16_16816(o[c + 1], pa, b1);
                }
            }
        }
        __syncthreads();
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
    bf16* o_lo = out + ((size_t)(start + q_off + r_lo) * q_heads + head) * HD;
    bf16* o_hi = out + ((size_t)(start + q_off + r_hi) * q_heads + head) * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        if (v_lo) *reinterpret_cast<uint32_t*>(o_lo + col) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (v_hi) *reinterpret_cast<uint32_t*>(o_hi + col) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

template <int HD>
static int launch_prefill(const void* q, const void* cache, const int* seg_info, const int* tiles,
                          int n_tiles, const int* block_table, int max_pages, int page_size, int q_heads,
                          int kv_heads, int window, float scale, void* out, cudaStream_t stream) {
    const size_t smem = (size_t)4 * kBN * HD * 2;
    static OncePerDevice configured;
    if (configured.first()) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_prefill_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("paged_attention_prefill: %s", cudaGetErrorString(e)); return (int)e; }
        configured.done();
    }
    launch_pdl(kPdlAttention, paged_attention_prefill_kernel<HD>, dim3(n_tiles, q_heads), dim3(kPfWarps * 32), smem, stream,
        (const bf16*)q, (const bf16*)cache, seg_info, tiles, block_table, max_pages, page_size, q_heads,
        kv_heads, window, scale * 1.4426950408889634f, (bf16*)out);
    return finish_launch("paged_attention_prefill");
}

}  // namespace tllm

using namespace tllm;

// seg_info: int[segments][4] = slot, first row, length, position of the first row.
// tiles: int[n_tiles][2] = segment, offset of the block's first query row in the segment.
extern "C" int tllm_paged_attention_prefill(
    const void* q, const void* cache, const int* seg_info, const int* tiles, int n_tiles,
    const int* block_table, int max_pages, int page_size, int q_heads, int kv_heads, int head_dim,
    int window, float scale, void* out, cudaStream_t stream) {
    TLLM_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
                 "paged_attention_prefill: %d query heads over %d key/value heads", q_heads, kv_heads);
    TLLM_REQUIRE(head_dim == 64 || head_dim == 128, "paged_attention_prefill: head_dim %d is not 64 or 128", head_dim);
    TLLM_REQUIRE(page_size > 0 && page_size % 16 == 0, "paged_attention_prefill: page size %d is no multiple of 16", page_size);
    TLLM_REQUIRE(n_tiles >= 0 && q_heads <= 65535, "paged_attention_prefill: bad grid");
    if (n_tiles == 0) return 0;
    if (head_dim == 64)
        return launch_prefill<64>(q, cache, seg_info, tiles, n_tiles, block_table, max_pages, page_size, q_heads,
                                  kv_heads, window, scale, out, stream);
    return launch_prefill<128>(q, cache, seg_info, tiles, n_tiles, block_table, max_pages, page_size, q_heads,
                               kv_heads, window, scale, out, stream);
}
