// y[M, N] = x[M, K] . W[N, K]^T in bfloat16 with float32 accumulation on the fifth-generation
// tensor cores (tcgen05), for the many-row products of a prefill step, with the SwiGLU of
// the feed-forward optionally fused into the epilogue.
//
// The reference calls cublasHgemm for these products and runs SwiGLU as a kernel of its own
// over the [tokens, 2 x intermediate] result (kernels/src/matmul_kernel_cuda.cu:83-91,
// kernels/src/swiglu_kernel_cuda.cu:7-27).
//
// The kernel is persistent: one block per SM walks over 128 x 256 tiles of y (row tiles
// fastest, so that blocks running at the same time share a slab of W in L2).  Warp 0 is the
// producer: one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a
// 128 x 64 slab of x and a 256 x 64 slab of W into a ring of four shared-memory stages and arms
// an mbarrier per stage with the expected byte count.  Warp 1 owns the tensor memory (all 512
// float32 columns of the SM's TMEM: two accumulators of 128 x 256) and issues the MMAs: one
// thread, four tcgen05.mma (128 x 256 x 16) per stage, shared-memory descriptors advanced by
// 32 bytes inside the swizzle atom; a tcgen05.commit hands the stage back to the producer when
// the tensor core has read it, another one hands the finished accumulator to the epilogue.
// Warps 2 to 5 are the epilogue: each thread owns one row of the tile, reads its accumulator
// row from TMEM 32 columns at a time (tcgen05.ld), writes bfloat16 to global memory and gives
// the accumulator back; meanwhile the MMAs of the next tile fill the other accumulator.  In
// SwiGLU mode the W slab is made of 128 gate rows and the 128 up rows that belong to them
// (two TMA boxes), so that columns j and 128 + j of the accumulator are gate and up of the
// same output: the epilogue writes silu(gate) * up, and the [tokens, 2 x intermediate] matrix
// never exists.
//
// Every wait on an mbarrier is bounded: when a limit runs out the block records a code in
// the error word the caller passed, stops issuing work, still waits (bounded) for the copies
// it has in flight, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

namespace tllm {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kStageBBytes = kBN * kBK * 2;
constexpr int kGemmThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr int kSpinLimit = 1 << 20;

__device__ __forceinline__ uint32_t cvta_shared(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(cvta_shared(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(cvta_shared(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(cvta_shared(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = cvta_shared(bar);
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

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
            cvta_shared(smem_dst)),
        "l"(map), "r"(cvta_shared(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major operand slab written by TMA with the 128-byte
// swizzle: rows of 128 bytes, groups of eight rows 1024 bytes apart (stride byte offset),
// leading byte offset unused (1), descriptor version 1 (Blackwell), layout type 2 (128B swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::f16: D float32 (bits 4-5 = 1), A and B bfloat16 (bits 7-9 and
// 10-12 = 1), both K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                     cvta_shared(bar))
                 : "memory");
}
// 32 consecutive float32 columns of this thread's TMEM lane (no wait: pair with tmem_ld_wait).
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
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

__device__ __forceinline__ void store_bf16x8(bf16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// Write 32 values of one output row starting at column col0 (vector stores where the row allows).
__device__ __forceinline__ void store_row32(bf16* row_ptr, int col0, int cols, const float* v) {
    if (col0 + 32 <= cols && (cols % 8) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) store_bf16x8(row_ptr + col0 + i, v + i);
    } else {
        for (int i = 0; i < 32; ++i)
            if (col0 + i < cols) row_ptr[col0 + i] = __float2bfloat16_rn(v[i]);
    }
}

// SWIGLU: W holds `half_n` gate rows and as many up rows, a column tile is 128 outputs and y is
// [M, half_n]; stacked ([gate; up]: the tile's gate and up rows are two boxes, accumulator columns
// 0..127 and 128..255) or interleaved by eight (eight gate rows, their eight up rows, ...: the
// tile is 256 neighbouring rows and a gate's up is eight columns further).  Otherwise a column
// tile is 256 outputs of N and y is [M, N].
// MT: row tiles of 128 per block.  MT = 1: two accumulators of 128 x 256 take turns, the
// epilogue of a tile overlaps the MMAs of the next, four stages of 48 KB.  MT = 2: the block
// owns 256 rows, both accumulators belong to one tile, every slab of W fetched from L2 feeds
// twice as many MMAs (32 KB of shared-memory fill per 128 x 256 x 64 instead of 48 KB), three
// stages of 64 KB; the epilogue is not overlapped.
template <bool SWIGLU, int MT>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    bf16* __restrict__ y, int M, int N, int K, int half_n, int interleaved, int tiles_m,
                    int tiles_n, int* __restrict__ error_word) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[4], empty_bar[4], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    // the dynamic window is not guaranteed to start on a 1024-byte boundary: round up
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    constexpr int kStages = MT == 1 ? 4 : 3, kNumBuf = MT == 1 ? 2 : 1;
    constexpr int kRows = kBM * MT, kStageABytes = kRows * kBK * 2, kStageBytes = kStageABytes + kStageBBytes;
    constexpr int kOutRowBytes = 64 * 2 + 16;                 // staging row of 64 outputs, padded
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* stage_out = tiles + (size_t)kStages * kStageBytes + (size_t)(warp & 3) * 32 * kOutRowBytes;
    const int k_blocks = (K + kBK - 1) / kBK;
    const int total_tiles = tiles_m * tiles_n;
    const int out_cols = SWIGLU ? half_n : N;
    constexpr int kColTile = SWIGLU ? 128 : kBN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);             // one arrival per epilogue warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {   // this warp owns the tensor memory from allocation to release
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         cvta_shared(&tmem_base_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* aborted = &abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            int it = 0;                               // k-blocks issued so far, over all tiles
            for (int t = blockIdx.x; t < total_tiles && !*aborted; t += gridDim.x) {
                const int tile_m = t % tiles_m, tile_n = t / tiles_m;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages && !mbar_wait(&empty_bar[s], ((it / kStages) - 1) & 1)) {
                        atomicExch(error_word, 1);
                        *aborted = 1;
                    }
                    if (*aborted) break;
                    unsigned char* a_dst = tiles + (size_t)s * kStageBytes;
                    unsigned char* b_dst = a_dst + kStageABytes;
                    mbar_expect_tx(&full_bar[s], kStageBytes);
                    tma_load_2d(a_dst, &map_x, kb * kBK, tile_m * kRows, &full_bar[s]);
                    if (SWIGLU && !interleaved) {
                        tma_load_2d(b_dst, &map_w, kb * kBK, tile_n * 128, &full_bar[s]);
                        tma_load_2d(b_dst + kStageBBytes / 2, &map_w, kb * kBK, half_n + tile_n * 128, &full_bar[s]);
                    } else {
                        tma_load_2d(b_dst, &map_w, kb * kBK, tile_n * kBN, &full_bar[s]);
                        tma_load_2d(b_dst + kStageBBytes / 2, &map_w, kb * kBK, tile_n * kBN + 128, &full_bar[s]);
                    }
                }
            }
            // on an abort: do not leave the block while copies into its shared memory are in flight
            if (*aborted) {
                const int first = it > kStages ? it - kStages : 0;
                for (int i = first; i < it; ++i) mbar_wait(&full_bar[i % kStages], (i / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(kBM, kBN);
            int it = 0, local = 0;
            for (int t = blockIdx.x; t < total_tiles && !*aborted; t += gridDim.x, ++local) {
                const int buf = local % kNumBuf;
                if (local >= kNumBuf && !mbar_wait(&acc_empty[buf], ((local / kNumBuf) - 1) & 1)) {
                    atomicExch(error_word, 4);
                    *aborted = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t tmem_acc = tmem_base + buf * kBN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(&full_bar[s], (it / kStages) & 1)) {
                        atomicExch(error_word, 2);
                        *aborted = 1;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = cvta_shared(tiles + (size_t)s * kStageBytes);
                    const uint32_t b_addr = a_addr + kStageABytes;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        const uint64_t b_desc = smem_desc_sw128(b_addr + k * 32);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint64_t a_desc = smem_desc_sw128(a_addr + mt * (kBM * kBK * 2) + k * 32);
                            umma_bf16(tmem_acc + mt * kBN, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty_bar[s]);      // the stage is free once these MMAs have read it
                }
                umma_commit(&acc_full[buf]);         // the accumulator is complete once all MMAs are done
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (four warps, one row per thread)
        const int quad = warp & 3;                   // a warp may read TMEM lanes 32 * (warp % 4) .. + 31
        int local = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
            const int buf = local % kNumBuf;
            const int tile_m = t % tiles_m, tile_n = t / tiles_m;
            const bool ready = mbar_wait(&acc_full[buf], (local / kNumBuf) & 1);
            if (!ready) {
                if (lane == 0) atomicExch(error_word, 3);
                *aborted = 1;
            }
            if (*aborted) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
                const int row0 = tile_m * kRows + mt * kBM + quad * 32;          // first row of this warp
                const uint32_t lane_addr = tmem_base + (buf + mt) * kBN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
                for (int c = 0; c < kColTile; c += 64) {                          // 64 output columns at a time
                    float v[64];
                    if (SWIGLU && interleaved) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {             // 64 accumulator columns: 32 outputs
                            uint32_t r0[32], r1[32];
                            tmem_ld32_issue(lane_addr + 2 * c + 64 * h, r0);
                            tmem_ld32_issue(lane_addr + 2 * c + 64 * h + 32, r1);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int gi = 16 * (i >> 3) + (i & 7);
                                const float g0 = __uint_as_float(r0[gi]), g1 = __uint_as_float(r1[gi]);
                                v[32 * h + i] = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(r0[gi + 8]);
                                v[32 * h + 16 + i] = __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(r1[gi + 8]);
                            }
                        }
                    } else if (SWIGLU) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t gr[32], ur[32];
                            tmem_ld32_issue(lane_addr + c + 32 * h, gr);
                            tmem_ld32_issue(lane_addr + 128 + c + 32 * h, ur);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const float g = __uint_as_float(gr[i]);
                                v[32 * h + i] = __fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(ur[i]);
                            }
                        }
                    } else {
                        uint32_t r0[32], r1[32];
                        tmem_ld32_issue(lane_addr + c, r0);
                        tmem_ld32_issue(lane_addr + c + 32, r1);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            v[i] = __uint_as_float(r0[i]);
                            v[32 + i] = __uint_as_float(r1[i]);
                        }
                    }
                    // through the warp's staging tile, so that a store instruction writes whole
                    // 128-byte lines (4 rows x 128 bytes) instead of 16 bytes in each of 32 rows
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 64; i += 8) store_bf16x8(reinterpret_cast<bf16*>(stage_out + lane * kOutRowBytes) + i, v + i);
                    __syncwarp();
                    const int col0 = tile_n * kColTile + c;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int piece = lane + 32 * j, r = piece >> 3, p16 = piece & 7;
                        const int row = row0 + r, col = col0 + p16 * 8;
                        if (row < M && col < out_cols) {
                            const uint4 val = *reinterpret_cast<const uint4*>(stage_out + r * kOutRowBytes + p16 * 16);
                            bf16* dst = y + (size_t)row * out_cols + col;
                            if (col + 8 <= out_cols && (out_cols % 8) == 0) {
                                *reinterpret_cast<uint4*>(dst) = val;
                            } else {
                                const bf16* e = reinterpret_cast<const bf16*>(&val);
                                for (int i = 0; i < 8; ++i)
                                    if (col + i < out_cols) dst[i] = e[i];
                            }
                        }
                    }
                }
            }
            // the accumulator may be overwritten once all four warps have read it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
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

// Tensor map of a row-major [rows, k] bfloat16 matrix for boxes of `box_rows` x 64 with 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long k, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            v = 148;
        return v;
    }();
    return n;
}

template <bool SWIGLU, int MT>
static int launch_tcgen05(const CUtensorMap& mx, const CUtensorMap& mw, void* y, int M, int N, int K, int half_n,
                          int interleaved, int* error_word, cudaStream_t stream) {
    const size_t smem = (size_t)(MT == 1 ? 4 : 3) * (kBM * MT * kBK * 2 + kStageBBytes) + 1024 + 4 * 32 * (64 * 2 + 16);
    static OncePerDevice configured;
    if (configured.first()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<SWIGLU, MT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("gemm_tcgen05: %s", cudaGetErrorString(e)); return (int)e; }
        configured.done();
    }
    const int out_cols = SWIGLU ? half_n : N;
    const int col_tile = SWIGLU ? 128 : kBN;
    const int tiles_n = (out_cols + col_tile - 1) / col_tile, tiles_m = (M + kBM * MT - 1) / (kBM * MT);
    const int total = tiles_m * tiles_n;
    const int grid = total < sm_count() ? total : sm_count();
    gemm_tcgen05_kernel<SWIGLU, MT><<<grid, kGemmThreads, smem, stream>>>(mx, mw, (bf16*)y, M, N, K, half_n, interleaved,
                                                                      tiles_m, tiles_n, error_word);
    return finish_launch("gemm_tcgen05");
}

}  // namespace tllm

using namespace tllm;

// y = x . w^T (y is [M, N]) or, with bit 1 of `swiglu`, y = silu(x . gate^T) * (x . up^T) (y is
// [M, N / 2]) for w = [gate; up], or with bit 4 as well for gate and up rows interleaved by eight.
// Bit 2 keeps blocks of 128 rows.  x [M, K], w [N, K] bfloat16 row-major, K a multiple of 8,
// operands 16-byte aligned.  `error_word` is a device int the kernel sets to a non-zero code if
// one of its bounded waits ran out (the result is then invalid); the caller clears and reads it.
extern "C" int tllm_gemm_tcgen05(const void* x, const void* w, void* y, int M, int N, int K, int swiglu,
                                 int* error_word, cudaStream_t stream) {
    TLLM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes");
    TLLM_REQUIRE(K % 8 == 0, "gemm_tcgen05: K = %d is no multiple of 8", K);
    TLLM_REQUIRE(!(swiglu & 1) || N % 2 == 0, "gemm_tcgen05: SwiGLU needs an even number of weight rows");
    const int interleaved = (swiglu & 4) ? 1 : 0;
    TLLM_REQUIRE(!interleaved || ((swiglu & 1) && N % 16 == 0),
                 "gemm_tcgen05: interleaved gate and up rows come in sixteens, N = %d", N);
    TLLM_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0,
                 "gemm_tcgen05: operands must be 16-byte aligned");
    TLLM_REQUIRE(error_word != nullptr, "gemm_tcgen05: no error word");
    CUtensorMap mx, mw;
    const bool tall = M > 128 && !(swiglu & 2) ;          // blocks of 256 rows once there are that many
    TLLM_REQUIRE(make_map(&mx, x, M, K, tall ? 2 * kBM : kBM) && make_map(&mw, w, N, K, 128),
                 "gemm_tcgen05: cuTensorMapEncodeTiled failed or is not available");
    if (swiglu & 1)
        return tall ? launch_tcgen05<true, 2>(mx, mw, y, M, N, K, N / 2, interleaved, error_word, stream)
                    : launch_tcgen05<true, 1>(mx, mw, y, M, N, K, N / 2, interleaved, error_word, stream);
    return tall ? launch_tcgen05<false, 2>(mx, mw, y, M, N, K, 0, 0, error_word, stream)
                : launch_tcgen05<false, 1>(mx, mw, y, M, N, K, 0, 0, error_word, stream);
}
