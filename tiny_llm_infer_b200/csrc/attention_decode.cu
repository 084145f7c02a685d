// Attention of single tokens (decode rows) over the paged cache, bfloat16, split over the
// keys of a request so that a handful of rows still fills the GPU.
//
// One block owns (row, key/value head, split): the query heads that share the key/value
// head form the rows of a 16-row tensor-core tile (the rest of the tile is zero), so keys
// and values are read from HBM once per group, not once per query head as the reference
// does (kernels/src/paged_attention_cuda.cu:70-120, one block per (token, head)).  Each of
// the four warps walks every fourth 16-key tile of the split: cp.async brings the tile's
// keys and values (one contiguous 16 x head_dim block of a page) into the warp's own
// double-buffered shared memory; scores are Q K^T on mma.sync, the softmax is online in
// float32 (base 2, scale folded in after the product), and P V accumulates in float32
// registers.  Warps are merged through shared memory; the block writes an unnormalised
// partial (and its maximum and sum) per split, and a second small kernel combines the
// splits in a fixed order.  With one split the block writes the result itself.
//
// Takes head widths 64 and 128, page sizes that are multiples of 16, groups of up to 16
// query heads per key/value head; anything else is refused (the caller then uses the
// general kernel).
#include "common.cuh"
#include "mma_tiles.cuh"

namespace tllm {

constexpr int kDecWarps = 4;
constexpr int kTileKeys = 16;
// Tiles of keys and values a warp has in its ring: one being multiplied, the others on their way.
// Measured at Qwen3-8B sizes, context 4096, whole decode steps: three stages (two tiles of 8 KB in
// flight per warp, 96 KB of shared memory and so two blocks per SM instead of three) take 4.17 ms
// at batch 8 and 10.09 at batch 64, two stages 4.14 and 9.92.
constexpr int kDecStages = 2;

template <int HD>
__global__ void __launch_bounds__(kDecWarps * 32)
paged_attention_decode_kernel(const bf16* q, const bf16* cache,
                              const int* __restrict__ positions, const int* __restrict__ token_slot,
                              const int* __restrict__ rows, const int* __restrict__ block_table,
                              int max_pages, int page_size, int q_heads, int kv_heads, int window,
                              float scale_log2e, int splits, float* __restrict__ part_o,
                              float* __restrict__ part_ml, bf16* __restrict__ out) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // The kernel after this one (the short one that combines the splits, which in its turn hides the
    // start of the product after it) may start early once every block has let it.
    TLLM_PDL_TRIGGER();
    constexpr int kChunks = HD / 8;                 // 16-byte chunks per row
    constexpr int kTileBytes = kTileKeys * HD * 2;  // one K or V tile
    const int split = blockIdx.x, g = blockIdx.y, ridx = blockIdx.z;
    const int r = rows ? rows[ridx] : ridx;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = q_heads / kv_heads;
    const int slot = token_slot[r];
    if (slot < 0) {
        TLLM_PDL_WAIT();
        if (splits == 1)                                     // else the combine kernel writes the zeros
            for (int i = threadIdx.x; i < group * HD; i += blockDim.x)
                out[((size_t)r * q_heads + g * group) * HD + i] = __float2bfloat16_rn(0.0f);
        return;
    }
    const int pos = positions[r];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int base = (lo / kTileKeys) * kTileKeys;
    const int n_keys = pos + 1 - base;
    int per = (n_keys + splits - 1) / splits;
    per = ((per + 4 * kTileKeys - 1) / (4 * kTileKeys)) * (4 * kTileKeys);   // whole rounds of the four warps
    const int k0 = base + split * per;
    const int k1 = min(pos + 1, k0 + per);
    const int lower = max(lo, k0), upper = k1 - 1;          // keys [lower, upper] count

    const int row_lo = lane >> 2, row_hi = row_lo + 8;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    unsigned char* my_smem = smem_raw + (size_t)warp * kDecStages * 2 * kTileBytes;   // stages x (K, V)
    const int* table = block_table + (size_t)slot * max_pages;
    const int first_tile = k0 / kTileKeys;
    const int last_tile = (k1 > k0) ? (k1 - 1) / kTileKeys : first_tile - 1;

    auto issue = [&](int tile, int stage) {
        const int key0 = tile * kTileKeys;
        const int page = table[key0 / page_size];
        const bool ok = page >= 0;
        const size_t off = ((size_t)(ok ? page : 0) * 2 * kv_heads + g) * page_size + (key0 % page_size);
        const bf16* kp = cache + off * HD;
        const bf16* vp = cache + (off + (size_t)kv_heads * page_size) * HD;
        const uint32_t ks = smem_u32(my_smem + (size_t)stage * 2 * kTileBytes);
        const uint32_t vs = ks + kTileBytes;
#pragma unroll
        for (int i = 0; i < (kTileKeys * kChunks) / 32; ++i) {
            const int c = lane + 32 * i, row = c / kChunks, chunk = c % kChunks;
            cp_async_16(ks + swizzled<HD>(row, chunk), kp + row * HD + chunk * 8, ok);
            cp_async_16(vs + swizzled<HD>(row, chunk), vp + row * HD + chunk * 8, ok);
        }
        cp_async_commit();
    };

    // every step commits one group (an empty one past the last tile), so that "all but the
    // newest kDecStages - 1 groups have landed" always means: the tile about to be used is there
    // Keys before the row's own position were written by earlier steps: a first tile that ends before
    // it is fetched (block table and all) while the kernel before this one, which writes the row's own
    // key and value and its query, may still be running.
    int tile = first_tile + warp;
    const bool early = kDecStages == 2 && tile <= last_tile && tile * kTileKeys + kTileKeys - 1 < pos;
    if (early) issue(tile, 0);
    TLLM_PDL_WAIT();
#pragma unroll
    for (int st = 0; st < kDecStages - 1; ++st) {
        if (early && st == 0) continue;
        if (tile + st * kDecWarps <= last_tile) issue(tile + st * kDecWarps, st);
        else cp_async_commit();
    }

    // ---- query fragments (rows = query heads of the group), read while the first tile is on its way
    const bf16* qrow = q + ((size_t)r * q_heads + (size_t)g * group) * HD;
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const int c0 = ks * 16 + (lane & 3) * 2;
        qa[ks][0] = row_lo < group ? *reinterpret_cast<const uint32_t*>(qrow + row_lo * HD + c0) : 0u;
        qa[ks][1] = row_hi < group ? *reinterpret_cast<const uint32_t*>(qrow + row_hi * HD + c0) : 0u;
        qa[ks][2] = row_lo < group ? *reinterpret_cast<const uint32_t*>(qrow + row_lo * HD + c0 + 8) : 0u;
        qa[ks][3] = row_hi < group ? *reinterpret_cast<const uint32_t*>(qrow + row_hi * HD + c0 + 8) : 0u;
    }

    for (int stage = 0; tile <= last_tile; tile += kDecWarps, stage = stage + 1 == kDecStages ? 0 : stage + 1) {
        {
            const int ahead = tile + (kDecStages - 1) * kDecWarps;
            const int into = stage == 0 ? kDecStages - 1 : stage - 1;      // the stage used in the step before
            if (ahead <= last_tile) issue(ahead, into);
            else cp_async_commit();
            cp_async_wait<kDecStages - 1>();
        }
        __syncwarp();
        const uint32_t ks_base = smem_u32(my_smem + (size_t)stage * 2 * kTileBytes);
        const uint32_t vs_base = ks_base + kTileBytes;

        // ---- S = Q K^T for 16 keys (two n-tiles of 8)
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
        const int mid = lane >> 3, mrow = lane & 7;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t kb[4];
            ldmatrix_x4(kb, ks_base + swizzled<HD>((mid >> 1) * 8 + mrow, 2 * ks + (mid & 1)));
            const uint32_t b0[2] = {kb[0], kb[1]}, b1[2] = {kb[2], kb[3]};
            mma_bf16_16816(s[0], qa[ks], b0);
            mma_bf16_16816(s[1], qa[ks], b1);
        }
        // ---- mask, online softmax (base 2)
        const int key_base = tile * kTileKeys + (lane & 3) * 2;
        float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = key_base + nt * 8 + e;
                const bool ok = j >= lower && j <= upper;
                s[nt][e] = ok ? s[nt][e] * scale_log2e : -INFINITY;
                s[nt][2 + e] = ok ? s[nt][2 + e] * scale_log2e : -INFINITY;
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
        float p[2][4];
        float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p[nt][e] = exp2f(s[nt][e] - ms_lo);
                p[nt][2 + e] = exp2f(s[nt][2 + e] - ms_hi);
                sum_lo += p[nt][e];
                sum_hi += p[nt][2 + e];
            }
        l_lo = l_lo * c_lo + sum_lo;
        l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
        }
        const uint32_t pa[4] = {pack_bf16(p[0][0], p[0][1]), pack_bf16(p[0][2], p[0][3]),
                                pack_bf16(p[1][0], p[1][1]), pack_bf16(p[1][2], p[1][3])};
        // ---- O += P V
#pragma unroll
        for (int c = 0; c < HD / 8; c += 2) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, vs_base + swizzled<HD>((mid & 1) * 8 + mrow, c + (mid >> 1)));
            const uint32_t b0[2] = {vb[0], vb[1]}, b1[2] = {vb[2], vb[3]};
            mma_bf16_16816(o[c], pa, b0);
            mma_bf16_16816(o[c + 1], pa, b1);
        }
        __syncwarp();
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    // ---- merge the four warps (shared memory is reused once every copy has landed)
    __syncthreads();
    float* os = reinterpret_cast<float*>(smem_raw);             // [warps][16][HD]
    float* ms = os + kDecWarps * 16 * HD;                       // [warps][16]
    float* ls = ms + kDecWarps * 16;                            // [warps][16]
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        float* w = os + (size_t)warp * 16 * HD;
        w[row_lo * HD + col] = o[i][0];
        w[row_lo * HD + col + 1] = o[i][1];
        w[row_hi * HD + col] = o[i][2];
        w[row_hi * HD + col + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
        ms[warp * 16 + row_lo] = m_lo; ms[warp * 16 + row_hi] = m_hi;
        ls[warp * 16 + row_lo] = l_lo; ls[warp * 16 + row_hi] = l_hi;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx - row * HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, ms[w * 16 + row]);
        float total = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float mw = ms[w * 16 + row];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mm);
            total += ls[w * 16 + row] * f;
            acc += os[((size_t)w * 16 + row) * HD + d] * f;
        }
        const int head = g * group + row;
        if (splits == 1) {
            out[((size_t)r * q_heads + head) * HD + d] = __float2bfloat16_rn(acc / total);
        } else {
            const size_t p_idx = ((size_t)ridx * q_heads + head) * splits + split;
            part_o[p_idx * HD + d] = acc;
            if (d == 0) { part_ml[p_idx * 2] = mm; part_ml[p_idx * 2 + 1] = total; }
        }
    }
}

// out[row, head, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits in index order.
template <int HD>
__global__ void paged_attention_combine_kernel(const float* part_o, const float* part_ml,
                                               const int* __restrict__ token_slot,
                                               const int* __restrict__ rows, int q_heads, int splits,
                                               bf16* __restrict__ out) {
    TLLM_PDL_ENTER();
    const int ridx = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    const int r = rows ? rows[ridx] : ridx;
    bf16* dst = out + ((size_t)r * q_heads + head) * HD;
    if (token_slot[r] < 0) { dst[d] = __float2bfloat16_rn(0.0f); return; }
    const size_t base = ((size_t)ridx * q_heads + head) * splits;
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    float total = 0.0f, acc = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = part_ml[(base + s) * 2];
        const float f = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
        total += part_ml[(base + s) * 2 + 1] * f;
        acc += part_o[(base + s) * HD + d] * f;
    }
    dst[d] = __float2bfloat16_rn(acc / total);
}

template <int HD>
static int launch_decode(const void* q, const void* cache, const int* positions, const int* token_slot,
                         const int* rows, int n_rows, const int* block_table, int max_pages,
                         int page_size, int q_heads, int kv_heads, int window, float scale, int splits,
                         float* part_o, float* part_ml, void* out, cudaStream_t stream) {
    const size_t smem = (size_t)kDecWarps * kDecStages * 2 * kTileKeys * HD * 2;
    static OncePerDevice configured;
    if (configured.first()) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_decode_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("paged_attention_decode: %s", cudaGetErrorString(e)); return (int)e; }
        configured.done();
    }
    const dim3 grid(splits, kv_heads, n_rows);
    // With at most a block per SM (one to four rows of Qwen3 sizes) the kernel starts while the one before
    // it still runs and has its first keys and values on their way when that one ends (a decode step of
    // Qwen3-8B sizes at batch 1: 3.33 instead of 3.38 ms); with more blocks than that the early ones
    // are in the way of the kernel before (batch 8: 4.12 instead of 4.08 ms).
    const long long blocks = (long long)splits * kv_heads * n_rows;
    const int cls = blocks <= sm_count_cached() ? kPdlAlways : kPdlAttention;
    launch_pdl(cls, paged_attention_decode_kernel<HD>, grid, dim3(kDecWarps * 32), smem, stream,
        (const bf16*)q, (const bf16*)cache, positions, token_slot, rows, block_table, max_pages, page_size,
        q_heads, kv_heads, window, scale * 1.4426950408889634f, splits, part_o, part_ml, (bf16*)out);
    int rc = finish_launch("paged_attention_decode");
    if (rc != 0 || splits == 1) return rc;
    launch_pdl(kPdlCombine, paged_attention_combine_kernel<HD>, dim3(n_rows, q_heads), dim3(HD), 0, stream,
        (const float*)part_o, (const float*) part_ml, token_slot, rows, q_heads, splits, (bf16*)out);
    return finish_launch("paged_attention_combine");
}

}  // namespace tllm

using namespace tllm;

// Scratch the caller provides when splits > 1:
//   part_o  float[n_rows * q_heads * splits * head_dim],  part_ml  float[n_rows * q_heads * splits * 2].
extern "C" int tllm_paged_attention_decode(
    const void* q, const void* cache, const int* positions, const int* token_slot, const int* rows,
    int n_rows, const int* block_table, int max_pages, int page_size, int q_heads, int kv_heads,
    int head_dim, int window, float scale, int splits, float* part_o, float* part_ml, void* out,
    cudaStream_t stream) {
    TLLM_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads / kv_heads <= 16,
                 "paged_attention_decode: %d query heads over %d key/value heads (at most 16 per group)",
                 q_heads, kv_heads);
    TLLM_REQUIRE(head_dim == 64 || head_dim == 128, "paged_attention_decode: head_dim %d is not 64 or 128", head_dim);
    TLLM_REQUIRE(page_size > 0 && page_size % 16 == 0, "paged_attention_decode: page size %d is no multiple of 16", page_size);
    TLLM_REQUIRE(splits >= 1 && splits <= 65535 && n_rows >= 0 && n_rows <= 65535 && kv_heads <= 65535,
                 "paged_attention_decode: bad grid");
    TLLM_REQUIRE(splits == 1 || (part_o && part_ml), "paged_attention_decode: %d splits need scratch", splits);
    if (n_rows == 0) return 0;
    if (head_dim == 64)
        return launch_decode<64>(q, cache, positions, token_slot, rows, n_rows, block_table, max_pages, page_size,
                                 q_heads, kv_heads, window, scale, splits, part_o, part_ml, out, stream);
    return launch_decode<128>(q, cache, positions, token_slot, rows, n_rows, block_table, max_pages, page_size,
                              q_heads, kv_heads, window, scale, splits, part_o, part_ml, out, stream);
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that must not allocate device memory (see tllm_noalloc.h for
// who they are and for the rules).  The partial results of the key splits go to the array
// below, which is part of the library's device image.  In host code the name
// `g_noalloc_scratch` is only a stand-in for the symbol, never a device address: handing it
// to a kernel would make the kernel fault, or, where the GPU can reach host memory, use the
// wrong memory without a word.  Its device address comes from cudaGetSymbolAddress, looked
// up once per device by the first call made while that device is current.
#include "tllm_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[TLLM_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the current device, or nullptr (error text set).
float* noalloc_scratch_address() {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
        set_error("paged_attention_decode_noalloc: cannot tell the current device (%s)",
                  e != cudaSuccess ? cudaGetErrorString(e) : "index out of range");
        return nullptr;
    }
    if (g_noalloc_scratch_addr[device] == nullptr) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
        if (e != cudaSuccess || addr == nullptr) {
            set_error("paged_attention_decode_noalloc: cudaGetSymbolAddress failed (%s)", cudaGetErrorString(e));
            return nullptr;
        }
        g_noalloc_scratch_addr[device] = static_cast<float*>(addr);
    }
    return g_noalloc_scratch_addr[device];
}
}  // namespace

extern "C" long long tllm_noalloc_scratch_needed(int n_rows, int q_heads, int head_dim, int splits) {
    if (splits <= 1 || n_rows <= 0 || q_heads <= 0 || head_dim <= 0) return 0;
    return (long long)n_rows * q_heads * splits * (head_dim + 2);
}

extern "C" int tllm_paged_attention_decode_noalloc(
    const void* q, const void* cache, const int* positions, const int* token_slot, const int* rows,
    int n_rows, const int* block_table, int max_pages, int page_size, int q_heads, int kv_heads,
    int head_dim, int window, float scale, int splits, void* out, cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && q_heads > 0 && head_dim > 0 && splits >= 1,
                 "paged_attention_decode_noalloc: bad sizes");
    const long long need = tllm_noalloc_scratch_needed(n_rows, q_heads, head_dim, splits);
    TLLM_REQUIRE(need <= (long long)TLLM_NOALLOC_SCRATCH_FLOATS,
                 "paged_attention_decode_noalloc: %d rows x %d heads x %d splits x (%d + 2) = %lld floats of "
                 "scratch exceed the built-in %u; use fewer splits or rows, or the entry point that takes "
                 "the caller's scratch", n_rows, q_heads, splits, head_dim, need,
                 (unsigned)TLLM_NOALLOC_SCRATCH_FLOATS);
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (splits > 1) {
        float* base = noalloc_scratch_address();
        if (base == nullptr) return -1;
        const long long n = (long long)n_rows * q_heads * splits;
        part_o = base;                       // [n][head_dim], each element written before it is read
        part_ml = base + n * head_dim;       // [n][2]
    }
    return tllm_paged_attention_decode(q, cache, positions, token_slot, rows, n_rows, block_table, max_pages,
                                       page_size, q_heads, kv_heads, head_dim, window, scale, splits, part_o,
                                       part_ml, out, stream);
}
