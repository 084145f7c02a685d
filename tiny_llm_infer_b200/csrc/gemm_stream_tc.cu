// y[M, N] = x[M, K] . W[N, K]^T for 9 to 128 rows of x (decoding many requests at once, short
// portions of prompts), bfloat16 with float32 accumulation on tcgen05 tensor cores.
//
// With so few rows the product is bound by reading W once from HBM, and a kernel that tiles y by
// rows of x has too few tiles to keep 148 SMs fetching.  Here the roles are swapped: the tensor
// core's M dimension (128 lanes of tensor memory) runs over 128 rows of W, its N dimension over
// the rows of x (padded to 32, 64 or 128), and the accumulator is y^T for that tile.  The K
// dimension of a tile is shared by the blocks of a thread-block cluster, each streaming its run
// of K through a ring of shared-memory stages (TMA, 128-byte swizzle; 16 KB of W and up to 16 KB
// of x per stage); at the end every block puts its partial accumulator into its own shared
// memory and the blocks add them up through distributed shared memory, each for its share of
// the rows of x, in the order of the ranks.  Nothing partial goes through global memory and no
// second kernel runs.  The cluster size is the caller's choice (1 to 8): it sets how many
// blocks there are for the SMs (tiles x cluster size), two of which fit an SM.
//
// Warp 0 is the producer (one thread), warp 1 owns the tensor memory and issues the MMAs (one
// thread), warps 2 to 5 read the accumulator (one row of W per thread) and write the result.
// SwiGLU mode: W holds gate and up rows interleaved by eight, a tile of 128 rows gives 64
// outputs silu(gate) * up, y is [M, N / 2].
//
// The kernel may be launched to start early (programmatic dependent launch): the producer
// fetches its first stages of W, which no kernel writes, before it waits for the kernel
// ahead, and only then the rows of x.
//
// Every wait on an mbarrier is bounded; a block whose wait ran out records a code in the error
// word, stops issuing work, waits (bounded) for its copies in flight, still meets the others at
// the cluster's barriers, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

namespace tllm {
namespace gst {

constexpr int kTileN = 128;                       // rows of W per tile = lanes of tensor memory
constexpr int kBK = 64;                           // K per stage: 128 bytes, one swizzle atom
constexpr int kWBytes = kTileN * kBK * 2;         // 16 KB
constexpr int kThreads = 192;
constexpr int kSpinLimit = 1 << 20;
constexpr int kMaxStages = 8;

__device__ __forceinline__ uint32_t sa(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(sa(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(sa(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = sa(bar);
    for (int spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
        "l"(map), "r"(sa(bar)), "r"(c0), "r"(c1)
        : "memory");
}
// K-major operand slab written by TMA with the 128-byte swizzle (rows of 128 bytes, groups of
// eight rows 1024 bytes apart; descriptor version 1, layout type 2).
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16: D float32, A and B bfloat16, both K-major, N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t id, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(sa(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, int rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, int rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(remote)
                 : "memory");
    return v;
}
// Four neighbouring outputs of a row of `cols` columns, starting at column col (a multiple of 4).
template <typename OutT>
__device__ __forceinline__ void store4(OutT* row, int col, int cols, const float (&v)[4]) {
    if (col + 4 <= cols && (cols & 3) == 0) {
        if constexpr (sizeof(OutT) == 4) {
            *reinterpret_cast<float4*>(row + col) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            uint2 raw;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
            h[0] = __floats2bfloat162_rn(v[0], v[1]);
            h[1] = __floats2bfloat162_rn(v[2], v[3]);
            *reinterpret_cast<uint2*>(row + col) = raw;
        }
    } else {
        for (int i = 0; i < 4; ++i)
            if (col + i < cols) row[col + i] = from_f32<OutT>(v[i]);
    }
}

// MB: rows of x the tile is padded to (the MMA's N).  A stage is 16 KB of W and MB x 128 bytes
// of x.  After the last MMA the stages' memory holds the partial accumulator as float32
// [MB][kTileN + 4] (rows of x outermost, so that the blocks' sums read consecutive words).
template <int MB, bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(kThreads)
gemm_stream_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      OutT* __restrict__ y, int M, int N, int K, int stages, int* __restrict__ error_word) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    constexpr int kXBytes = MB * kBK * 2, kStageBytes = kWBytes + kXBytes;
    constexpr int kPartStride = kTileN + 4;
    constexpr uint32_t kCols = MB < 32 ? 32 : MB;            // tensor-memory columns: a power of two, at least 32
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t tiles_s = sa(tiles);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int splits = gridDim.x, rank = (int)cluster_rank(), tile = blockIdx.y;
    const int k_blocks = (K + kBK - 1) / kBK;
    const int per = (k_blocks + splits - 1) / splits;
    const int kb0 = rank * per, kb1 = min(k_blocks, kb0 + per);      // this block's run of K (may be empty)
    const int n_kb = kb1 > kb0 ? kb1 - kb0 : 0;

    asm volatile("griddepcontrol.launch_dependents;\n" ::);
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sa(&tmem_slot)), "r"(kCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_slot;
    volatile int* aborted = &abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            // W first, for as many stages as there are: nothing before this kernel writes it
            const int ahead = min(stages, n_kb);
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full_bar[i], kStageBytes);
                tma_load_2d(tiles_s + i * kStageBytes, &map_w, (kb0 + i) * kBK, tile * kTileN, &full_bar[i]);
            }
            asm volatile("griddepcontrol.wait;\n" ::: "memory");        // x comes from the kernel ahead
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(tiles_s + i * kStageBytes + kWBytes, &map_x, (kb0 + i) * kBK, 0, &full_bar[i]);
            // (stage and parity are counted along: a division per step is a good part of what a
            // step costs the one thread that issues it)
            int it = ahead, s = ahead == stages ? 0 : ahead;
            uint32_t parity = 0;
            bool failed = false;
            for (; it < n_kb; ++it) {
                if (!mbar_wait(&empty_bar[s], parity)) {
                    atomicExch(error_word, 21);
                    *aborted = 1;
                    failed = true;
                    break;
                }
                mbar_expect_tx(&full_bar[s], kStageBytes);
                tma_load_2d(tiles_s + s * kStageBytes, &map_w, (kb0 + it) * kBK, tile * kTileN, &full_bar[s]);
                tma_load_2d(tiles_s + s * kStageBytes + kWBytes, &map_x, (kb0 + it) * kBK, 0, &full_bar[s]);
                if (++s == stages) { s = 0; parity ^= 1; }
            }
            if (failed) {          // do not leave while copies into this block's shared memory are in flight
                const int first = it > stages ? it - stages : 0;
                for (int i = first; i < it; ++i) mbar_wait(&full_bar[i % stages], (i / stages) & 1);
            }
        } else {
            asm volatile("griddepcontrol.wait;\n" ::: "memory");
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (one thread)
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        if (lane == 0) {
            constexpr uint32_t id = idesc(kTileN, MB < 16 ? 16 : MB);
            int s = 0;
            uint32_t parity = 0;
            for (int it = 0; it < n_kb; ++it) {
                if (!mbar_wait(&full_bar[s], parity)) {        // also how this thread learns that the producer gave up
                    atomicExch(error_word, 22);
                    *aborted = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t w_addr = tiles_s + s * kStageBytes, x_addr = w_addr + kWBytes;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)
                    umma(tmem, desc_sw128(w_addr + k * 32), desc_sw128(x_addr + k * 32), id, (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);
                if (++s == stages) { s = 0; parity ^= 1; }
            }
            umma_commit(&acc_full);                  // all MMAs of this block have completed (also when there were none)
        }
    } else {
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
    }

    // ---------------------------------------------------------------- partial accumulator -> shared memory
    float* part = reinterpret_cast<float*>(tiles);             // [MB][kPartStride], over the stages
    if (warp >= 2) {
        const int quad = warp & 3, n = quad * 32 + lane;       // a warp reads lanes 32 * (warp % 4) .. + 31
        if (!mbar_wait(&acc_full, 0)) {
            if (lane == 0) atomicExch(error_word, 23);
            *aborted = 1;
        }
        const bool ok = !__any_sync(0xffffffffu, *aborted != 0);     // a warp takes one way
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < MB; c += 32) {
            uint32_t r[32];
            if (ok && n_kb > 0) {
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + c, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (c + i < MB) part[(c + i) * kPartStride + n] = __uint_as_float(r[i]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kCols) : "memory");
    }
    cluster_sync();                                            // every block's partial sums are in place

    // ---------------------------------------------------------------- sums over the cluster, this block's rows of x
    // Rank r sums the rows m = r, r + splits, ... of x.  A thread takes four neighbouring weight
    // rows of one m at a time and asks all ranks for them before it adds (in the order of the
    // ranks), so that the remote loads' latencies overlap.
    if (warp >= 2 && !*aborted) {
        const int t = threadIdx.x - 64;                        // 0..127
        const uint32_t part_s = sa(part);
        const int my_rows = M > rank ? (M - rank + splits - 1) / splits : 0;
        if (SWIGLU) {
            // outputs 4 j4 .. 4 j4 + 3 of the tile's 64: gate rows 16 (j4 / 2) + 4 (j4 % 2) .. + 3, up rows eight further
            const int out_cols = N / 2;
            for (int c = t; c < my_rows * 16; c += 128) {
                const int m = rank + (c >> 4) * splits, j4 = c & 15;
                const int gate = 16 * (j4 >> 1) + 4 * (j4 & 1);
                float4 g[8], u[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    if (r < splits) {
                        g[r] = ld_cluster_f32x4(part_s + (m * kPartStride + gate) * 4, r);
                        u[r] = ld_cluster_f32x4(part_s + (m * kPartStride + gate + 8) * 4, r);
                    }
                }
                float4 gs = g[0], us = u[0];
#pragma unroll
                for (int r = 1; r < 8; ++r) {
                    if (r < splits) {
                        gs.x += g[r].x; gs.y += g[r].y; gs.z += g[r].z; gs.w += g[r].w;
                        us.x += u[r].x; us.y += u[r].y; us.z += u[r].z; us.w += u[r].w;
                    }
                }
                const float v[4] = {__fdividef(gs.x, 1.0f + __expf(-gs.x)) * us.x, __fdividef(gs.y, 1.0f + __expf(-gs.y)) * us.y,
                                    __fdividef(gs.z, 1.0f + __expf(-gs.z)) * us.z, __fdividef(gs.w, 1.0f + __expf(-gs.w)) * us.w};
                store4(y + (size_t)m * out_cols, tile * (kTileN / 2) + 4 * j4, out_cols, v);
            }
        } else {
            for (int c = t; c < my_rows * 32; c += 128) {
                const int m = rank + (c >> 5) * splits, n4 = c & 31;
                float4 a[8];
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    if (r < splits) a[r] = ld_cluster_f32x4(part_s + (m * kPartStride + 4 * n4) * 4, r);
                float4 acc = a[0];
#pragma unroll
                for (int r = 1; r < 8; ++r)
                    if (r < splits) { acc.x += a[r].x; acc.y += a[r].y; acc.z += a[r].z; acc.w += a[r].w; }
                const float v[4] = {acc.x, acc.y, acc.z, acc.w};
                store4(y + (size_t)m * N, tile * kTileN + 4 * n4, N, v);
            }
        }
    }
    cluster_sync();                                            // nobody leaves while its shared memory is read
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// [rows, k] bfloat16 row-major, boxes of box_rows x 64, 128-byte swizzle; what lies outside reads as zero.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long k, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MB, bool SWIGLU, typename OutT>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* y, int M, int N, int K, int splits,
                  int* error_word, cudaStream_t stream) {
    constexpr int kStageBytes = kWBytes + MB * kBK * 2;
    // two blocks per SM: half of the 227 KB each, less the static part and the alignment slack
    static const int knob = [] { const char* v = getenv("TLLM_GST_STAGES"); return v != nullptr ? atoi(v) : 0; }();
    int stages = (112 * 1024 - 2048) / kStageBytes;
    if (knob > 0) stages = knob;                      // for measurements: more stages, one block per SM
    if (stages > kMaxStages) stages = kMaxStages;
    while ((size_t)stages * kStageBytes > 220 * 1024) --stages;
    size_t smem = (size_t)stages * kStageBytes;
    const size_t part_bytes = (size_t)MB * (kTileN + 4) * 4;
    if (smem < part_bytes) smem = part_bytes;
    smem += 1024;
    static OncePerDevice configured;
    if (configured.first()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_tc_kernel<MB, SWIGLU, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
        if (e != cudaSuccess) { set_error("gemm_stream_tc: %s", cudaGetErrorString(e)); return (int)e; }
        configured.done();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, (N + kTileN - 1) / kTileN);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_tc_kernel<MB, SWIGLU, OutT>, mw, mx, (OutT*)y, M, N, K, stages,
                                       error_word);
    if (e != cudaSuccess) { set_error("gemm_stream_tc: %s", cudaGetErrorString(e)); return (int)e; }
    return finish_launch("gemm_stream_tc");
}

}  // namespace gst
}  // namespace tllm

using namespace tllm;

// y = x . w^T for 1 <= M <= 128 rows: x [M, K], w [N, K] bfloat16 row-major, K a multiple of 8,
// operands 16-byte aligned; y [M, N] bfloat16 (out_f32 = 0) or float32.  With `swiglu` w holds
// gate and up rows interleaved by eight (N a multiple of 16) and y is [M, N / 2] =
// silu(x . gate^T) * (x . up^T).  `splits` (1 to 8) blocks share the K of a tile as one cluster;
// each gets at least one stage of 64.  `error_word`: device int, set non-zero when a bounded
// wait ran out (the result is then invalid).
extern "C" int tllm_gemm_stream_tc(const void* x, const void* w, void* y, int M, int N, int K, int swiglu, int out_f32,
                                   int splits, int* error_word, cudaStream_t stream) {
    TLLM_REQUIRE(M >= 1 && M <= 128 && N > 0 && K > 0, "gemm_stream_tc: M = %d outside 1..128 (N %d, K %d)", M, N, K);
    TLLM_REQUIRE(K % 8 == 0, "gemm_stream_tc: K = %d is no multiple of 8", K);
    TLLM_REQUIRE(!swiglu || N % 16 == 0, "gemm_stream_tc: interleaved gate and up rows come in sixteens, N = %d", N);
    TLLM_REQUIRE(!(swiglu && out_f32), "gemm_stream_tc: the fused activation writes bfloat16");
    TLLM_REQUIRE(splits >= 1 && splits <= 8 && splits <= (K + 63) / 64, "gemm_stream_tc: %d splits (1 to 8, at most K / 64)",
                 splits);
    TLLM_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0,
                 "gemm_stream_tc: operands must be 16-byte aligned");
    TLLM_REQUIRE(error_word != nullptr, "gemm_stream_tc: no error word");
    const int mb = M <= 32 ? 32 : M <= 64 ? 64 : 128;
    CUtensorMap mw, mx;
    TLLM_REQUIRE(gst::make_map(&mw, w, N, K, gst::kTileN) && gst::make_map(&mx, x, M, K, mb),
                 "gemm_stream_tc: cuTensorMapEncodeTiled failed or is not available");
#define GST_LAUNCH(MB)                                                                                          \
    do {                                                                                                        \
        if (swiglu) return gst::launch<MB, true, bf16>(mw, mx, y, M, N, K, splits, error_word, stream);         \
        if (out_f32) return gst::launch<MB, false, float>(mw, mx, y, M, N, K, splits, error_word, stream);      \
        return gst::launch<MB, false, bf16>(mw, mx, y, M, N, K, splits, error_word, stream);                    \
    } while (0)
    if (mb == 32) GST_LAUNCH(32);
    if (mb == 64) GST_LAUNCH(64);
    GST_LAUNCH(128);
#undef GST_LAUNCH
}
