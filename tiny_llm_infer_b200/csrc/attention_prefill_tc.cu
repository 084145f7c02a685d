// Attention of prompt portions over the paged cache on the fifth-generation tensor cores:
// queries (TMA), keys and values (cp.async) come into shared memory, tcgen05.mma computes S = Q K^T and
// O += P V with S, P and O in tensor memory, and the softmax runs on what tcgen05.ld reads back.
// Head width 128, bfloat16, pages of a multiple of 16 tokens.
//
// (The reference treats each prompt token as a decode query of its own,
// kernels/src/paged_attention_cuda.cu:70-120; the mma.sync version of this kernel is
// attention_prefill.cu, which stays for head width 64 and as the comparison in the tests.)
//
// A block owns TWO tiles of 128 query rows that read the same keys and values, so that every
// key tile fetched from L2 serves 256 rows (with one tile per block the kernel ran at the L2's
// bandwidth): two query heads of one key/value head at the same 128 positions where the group
// is even, else two consecutive blocks of 128 positions of one head.  It walks the request's
// keys in tiles of 64; a tile outside one of the two ranges is skipped for that one.
//   warps 2-3 copy the key and value tiles with 16-byte cp.async into the layout the MMAs read
//             (the copy engine takes some 300 cycles per box whatever its size, and pages of 16
//             keys make for small boxes), into rings of five key and five value tiles; the block
//             table is looked up for 32 groups of 16 keys at a time.  The two 128 x 128 query
//             tiles come by TMA, once.
//   warps 1, 0  issue the MMAs of the first and second query tile (one elected thread each; an
//             issue costs the thread some 50 cycles, a look at a barrier some 200, and one thread
//             for both tiles was the bottleneck).  S[128 x 64] = Q K^T (8 x tcgen05.mma
//             128x64x16, both operands K-major in shared memory) goes into one of two S buffers,
//             one key tile ahead of the softmax (and only after the P V product that read that
//             buffer has completed: MMAs into different accumulators are not ordered).  Once the
//             softmax has put P into tensor memory (over the S it read), O[128 x 128] += P V
//             (4 x tcgen05.mma 128x128x16 with A from tensor memory and V as it lies in the
//             cache: an MN-major operand).  tcgen05.commit frees the stages and tells the
//             softmax warps.
//   warps 4-7, 8-11  softmax of the first and second query tile, one row per thread (TMEM lane =
//             row): read S, mask by the row's position and window where the tile needs it,
//             softmax in base 2 in float32 against a reference maximum that is only raised when
//             a tile exceeds it by more than 2^8 (then O, which stays in tensor memory, and the
//             row sum are scaled down: rare after the first tiles), write P as bfloat16 back
//             into tensor memory.  At the end O / sum goes through shared memory to whole-line
//             stores.
// One block per SM (224 KB of shared memory, all 512 TMEM columns).  Every mbarrier wait is
// bounded; on a timeout the block sets the caller's error word, stops, waits (bounded) for
// copies and MMAs in flight, frees its tensor memory and returns.
#include <climits>
#include <cuda.h>

#include "common.cuh"

namespace tllm {
namespace pftc {

constexpr int kHD = 128, kBM = 128, kBN = 64;
constexpr int kQBytes = kBM * kHD * 2;            // 32 KB: two column halves of [128 rows x 128 B]
constexpr int kKBytes = kBN * kHD * 2;            // 16 KB: two column halves of [64 keys x 128 B]
constexpr int kVBytes = kKBytes;
constexpr int kStages = 5;                        // of the key ring and of the value ring
constexpr int kTilesBytes = 2 * kQBytes + kStages * (kKBytes + kVBytes);   // 224 KB
constexpr int kSmemBytes = kTilesBytes + 512;     // + barriers and the TMEM slot
constexpr int kThreads = 384;
// query tile x: S buffers (and P over them) at columns x * 128 + {0, 64}, O at 256 + x * 128
constexpr uint32_t kTmemCols = 512;
constexpr float kRaise = 8.0f;                    // the reference maximum follows only beyond 2^8
constexpr int kSpinLimit = 1 << 20;

__device__ __forceinline__ uint32_t sa(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(sa(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(sa(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(sa(bar)) : "memory");
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
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
            smem_dst),
        "l"(map), "r"(sa(bar)), "r"(c0), "r"(c1)
        : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, eight-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand, 128-byte swizzle: a row of 128 bytes holds 64 consecutive MN elements of one
// k; eight k's form a 1024-byte group (stride byte offset), the next 64 MN elements lie
// `mn_block_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t mn_block_bytes) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(mn_block_bytes >> 4) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: float32 accumulator, bfloat16 operands, A K-major, B K-major
// (b_mn_major = 0) or MN-major (1), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t id, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(id), "r"(acc)
        : "memory");
}
// A from tensor memory (lane = row, two bfloat16 per 32-bit column), B from shared memory.
__device__ __forceinline__ void umma_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t id, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(id), "r"(acc)
        : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(sa(bar))
                 : "memory");
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct Barriers {
    uint64_t q_full, full[kStages], k_empty[kStages], v_empty[kStages];
    uint64_t s_full[2][2], p_full[2][2], o_full[2], o_done[2], drain[2];
    uint32_t tmem_slot;
    int abort_flag;
};
static_assert(sizeof(Barriers) <= 512, "barrier block");

// One of the block's two query tiles: `n` key tiles from `kt_first` on (n = 0: no such tile).
struct QTile {
    int head, q_off, rows, first_pos, last_pos, kt_first, n;
};

__global__ void __launch_bounds__(kThreads, 1)
paged_attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const bf16* __restrict__ cache,
                                  const int* __restrict__ seg_info, const int* __restrict__ tiles,
                                  const int* __restrict__ block_table, int max_pages, int page_size, int q_heads,
                                  int kv_heads, int window, float scale_log2e, int pair_heads,
                                  bf16* __restrict__ out, int splits, float* __restrict__ part_o,
                                  float* __restrict__ part_ml, int* __restrict__ error_word) {
    extern __shared__ __align__(1024) unsigned char smem[];
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kTilesBytes);
    volatile int* aborted = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_s = sa(smem), k_s = q_s + 2 * kQBytes, v_s = k_s + kStages * kKBytes;

    // blocks start in the order of the tile list (the caller puts the longest first), heads fastest
    const int seg = tiles[2 * blockIdx.y], q_off0 = tiles[2 * blockIdx.y + 1];
    const int slot = seg_info[4 * seg], start = seg_info[4 * seg + 1];
    const int len = seg_info[4 * seg + 2], pos0 = seg_info[4 * seg + 3];
    QTile qt[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        QTile& t = qt[x];
        t.head = pair_heads ? 2 * blockIdx.x + x : blockIdx.x;
        t.q_off = pair_heads ? q_off0 : q_off0 + x * kBM;
        t.rows = min(kBM, len - t.q_off);
        t.first_pos = pos0 + t.q_off;
        t.last_pos = t.first_pos + t.rows - 1;
        const int lo = (window > 0 && t.first_pos - window + 1 > 0) ? t.first_pos - window + 1 : 0;
        t.kt_first = lo / kBN;
        t.n = t.rows > 0 ? t.last_pos / kBN - t.kt_first + 1 : 0;
    }
    const int g = qt[0].head / (q_heads / kv_heads);           // both tiles read this key/value head
    const int last_pos = max(qt[0].last_pos, qt[1].rows > 0 ? qt[1].last_pos : 0);
    // the key tiles some query tile of the block reads: [kt_lo, kt_lo + n_tiles)
    auto block_range = [&](int& lo, int& end) {
        lo = INT_MAX, end = 0;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            if (qt[x].n > 0) {
                lo = min(lo, qt[x].kt_first);
                end = max(end, qt[x].kt_first + qt[x].n);
            }
        }
    };
    int kt_lo, kt_end;
    block_range(kt_lo, kt_end);
    if (splits > 1) {
        // this block takes the blockIdx.z-th of `splits` equal runs of those tiles and leaves
        // unnormalised partial results; a query tile may have nothing in the run
        const int part = (kt_end - kt_lo + splits - 1) / splits;
        const int a = kt_lo + (int)blockIdx.z * part, b = min(kt_end, a + part);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            QTile& t = qt[x];
            if (t.n > 0) {
                const int na = max(t.kt_first, a), nb = min(t.kt_first + t.n, b);
                t.kt_first = na;
                t.n = max(0, nb - na);
            }
        }
        block_range(kt_lo, kt_end);
    }
    const int n_tiles = kt_end > kt_lo ? kt_end - kt_lo : 0;
    // partial results of row r of query tile t: O at part_o + index * kHD, (reference maximum, sum) at part_ml + index * 2
    auto part_index = [&](const QTile& t, int r) -> size_t {
        return ((size_t)(start + t.q_off + r) * q_heads + t.head) * splits + blockIdx.z;
    };
    if (splits > 1 && warp >= 4) {                            // a tile with no key in this run says so
        const QTile& t = qt[(warp - 4) >> 2];
        const int r = (warp & 3) * 32 + lane;
        if (t.n == 0 && r < t.rows) {
            float* ml = part_ml + part_index(t, r) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.0f;
        }
    }
    if (n_tiles == 0) return;                                 // (only with splits) nothing for either tile

    if (threadIdx.x == 0) {
        if (q_s & 1023) atomicExch(error_word, 9);         // operand tiles need a 1024-byte aligned window
        mbar_init(&bars->q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bars->full[s], 2);                   // two copying warps
            mbar_init(&bars->k_empty[s], 2);                // two MMA warps
            mbar_init(&bars->v_empty[s], 2);
        }
        for (int x = 0; x < 2; ++x) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(&bars->s_full[x][b], 1);
                mbar_init(&bars->p_full[x][b], 4);          // one arrival per softmax warp
            }
            mbar_init(&bars->o_full[x], 1);
            mbar_init(&bars->o_done[x], 1);
        }
        mbar_init(&bars->drain[0], 1);
        mbar_init(&bars->drain[1], 1);
        bars->abort_flag = (q_s & 1023) ? 1 : 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sa(&bars->tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = bars->tmem_slot;

    if (warp < 2) {
        // -------------------------------------------------------------------- MMA issuers (and the query tiles)
        // Warp 1 issues for the first query tile, warp 0 for the second: an issue costs the thread
        // some 50 cycles and a wait on a barrier some 200, so one thread for both tiles was the
        // kernel's bottleneck.  The whole warp runs the loop, so that addresses and descriptors
        // are warp-uniform values; one elected lane issues the MMAs and commits (a commit covers
        // that thread's MMAs).
        const int x = warp == 1 ? 0 : 1;
        const QTile t = x ? qt[1] : qt[0];
        if (warp == 0 && lane == 0 && !*aborted) {           // query tiles, by TMA, once
            mbar_expect_tx(&bars->q_full, ((qt[0].n > 0) + (qt[1].n > 0)) * kQBytes);
#pragma unroll
            for (int y = 0; y < 2; ++y) {
                if (qt[y].n == 0) continue;
                tma_load_2d(q_s + y * kQBytes, &map_q, qt[y].head * kHD, start + qt[y].q_off, &bars->q_full);
                tma_load_2d(q_s + y * kQBytes + kQBytes / 2, &map_q, qt[y].head * kHD + 64, start + qt[y].q_off,
                            &bars->q_full);
            }
        }
        __syncwarp();
        const bool leader = elect_one();
        constexpr uint32_t id_s = idesc(kBM, kBN, 0), id_o = idesc(kBM, kHD, 1);
        const uint32_t q_addr = q_s + x * kQBytes, tmem_s = tmem + x * 128, tmem_o = tmem + 256 + x * 128;
        auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity));
        };
        // S of this query tile for the block's key tile j (copied in step j); 0 or an error code
        auto issue_s = [&](int j) -> int {
            const int jx = kt_lo + j - t.kt_first, s = j % kStages;
            if (jx >= 0 && jx < t.n) {
                // S(jx) goes where PV(jx-2) read its P: that one has to have completed
                if (jx >= 2 && !wait_all(&bars->o_full[x], (jx - 2) & 1)) return 5;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d = tmem_s + (jx & 1) * kBN, k_addr = k_s + s * kKBytes;
#pragma unroll
                for (int k = 0; k < kHD / 16; ++k) {        // S = Q K^T over the head width
                    const uint32_t half = k >> 2, kk = k & 3;
                    const uint64_t da = desc_k_major(q_addr + half * (kQBytes / 2) + kk * 32);
                    const uint64_t db = desc_k_major(k_addr + half * (kKBytes / 2) + kk * 32);
                    if (leader) umma(d, da, db, id_s, k > 0 ? 1u : 0u);
                }
                if (leader) umma_commit(&bars->s_full[x][jx & 1]);
            }
            if (leader) umma_commit(&bars->k_empty[s]);
            return 0;
        };
        // the query tiles have to be there before anything is issued (and before warp 0 may leave)
        int err = wait_all(&bars->q_full, 0) ? 0 : 3;
        if (!err && !wait_all(&bars->full[0], 0)) err = 4;
        if (!err && !__any_sync(0xffffffffu, *aborted != 0)) err = issue_s(0);
        for (int j = 0; j < n_tiles && !err; ++j) {
            if (__any_sync(0xffffffffu, *aborted != 0)) break;
            // step j+1 brought K(j+1) and V(j)
            if (!wait_all(&bars->full[(j + 1) % kStages], ((j + 1) / kStages) & 1)) { err = 4; break; }
            if (j + 1 < n_tiles && (err = issue_s(j + 1)) != 0) break;
            const int jx = kt_lo + j - t.kt_first, s = j % kStages;
            if (jx >= 0 && jx < t.n) {
                if (!wait_all(&bars->p_full[x][jx & 1], (jx >> 1) & 1)) { err = 7; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t p = tmem_s + (jx & 1) * kBN, v_addr = v_s + s * kVBytes;
#pragma unroll
                for (int k = 0; k < kBN / 16; ++k) {        // O += P V over the tile's keys
                    const uint64_t db = desc_mn_major(v_addr + k * 2048, kVBytes / 2);
                    if (leader) umma_ta(tmem_o, p + k * 8, db, id_o, (jx > 0 || k > 0) ? 1u : 0u);
                }
                if (leader) {
                    umma_commit(&bars->o_full[x]);
                    if (jx == t.n - 1) umma_commit(&bars->o_done[x]);
                }
            }
            if (leader) umma_commit(&bars->v_empty[s]);
        }
        if (err && leader) { atomicExch(error_word, err); *aborted = 1; }
        __syncwarp();
        if (__any_sync(0xffffffffu, *aborted != 0) && leader) {   // tensor memory is freed below: let the MMAs end first
            umma_commit(&bars->drain[x]);
            mbar_wait(&bars->drain[x], 0);
        }
        __syncwarp();
    } else if (warp == 2 || warp == 3) {
        // -------------------------------------------------------------------- key and value tiles (cp.async)
        // Pages are 16 keys or more apart in memory, and the copy engine takes some 300 cycles per
        // box whatever its size, so the tiles are gathered with 16-byte asynchronous copies into
        // the layout the MMAs read (rows of 128 bytes per column half, 16-byte chunks swizzled by
        // the row).  Warp w - 2 copies keys 32 (w - 2) .. +31 of every tile: an instruction moves
        // two whole rows of 256 bytes, 16 lanes each.  The cache rows of the warp's next 32 groups
        // of 16 keys (16 tiles) are looked up at once, one group per lane, and handed out by
        // shuffle; the 32 after them are fetched while these are in use.
        const int w = warp - 2;
        const int* table = block_table + (size_t)slot * max_pages;
        const char* cache_b = reinterpret_cast<const char*>(cache);
        const int v_off = kv_heads * page_size;              // from a key's row to its value's
        auto lookup = [&](int chunk) -> int {                // row of K of this lane's group, -1: none
            const int idx = chunk * 32 + lane;
            const int key0 = ((kt_lo + (idx >> 1)) * 4 + w * 2 + (idx & 1)) * 16;
            if (key0 > last_pos) return -1;
            const int page = table[key0 / page_size];
            return page < 0 ? -1 : (int)(((long long)page * 2 * kv_heads + g) * page_size + key0 % page_size);
        };
        int rows0 = lookup(0), rows1 = -1;                   // chunks of even and odd number
        auto copy_tile = [&](int j, int value, uint32_t dst) {
            const int held = ((j >> 4) & 1) ? rows1 : rows0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int base = __shfl_sync(0xffffffffu, held, (j & 15) * 2 + h);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int in_grp = 2 * i + (lane >> 4), key = w * 32 + h * 16 + in_grp, c = lane & 15;
                    const long long row = (long long)base + in_grp + (value ? v_off : 0);
                    const char* src = base < 0 ? cache_b : cache_b + row * (kHD * 2) + c * 16;
                    const uint32_t d = dst + (c >> 3) * (kKBytes / 2) + key * 128 + (((c & 7) ^ (key & 7)) << 4);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src),
                                 "r"(base < 0 ? 0 : 16)
                                 : "memory");                // zero-filled where the request holds no key
                }
            }
        };
        // Step s copies K(s) and V(s-1) as one group and publishes them on full[s % kStages];
        // kInFlight groups are under way per thread.
        constexpr int kInFlight = 3;
        auto publish = [&](int st) {      // the step's copies of this warp have landed: tell the MMA thread
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->full[st % kStages]);
        };
        bool stop = __any_sync(0xffffffffu, *aborted != 0);
        int committed = 0, published = 0;
        for (int st = 0; st <= n_tiles && !stop; ++st) {
            const int jk = st, jv = st - 1;
            bool ok = true;
            if (jk < n_tiles) {
                if ((jk & 15) == 1) {                        // values have left the chunk before: fetch the next
                    const int next = lookup((jk >> 4) + 1);
                    if ((jk >> 4) & 1) rows0 = next; else rows1 = next;
                }
                if (jk >= kStages && lane == 0) ok = mbar_wait(&bars->k_empty[jk % kStages], ((jk / kStages) - 1) & 1);
            }
            if (ok && jv >= kStages && lane == 0) ok = mbar_wait(&bars->v_empty[jv % kStages], ((jv / kStages) - 1) & 1);
            if (!ok) { atomicExch(error_word, 1); *aborted = 1; }
            if (__any_sync(0xffffffffu, !ok || *aborted != 0)) { stop = true; break; }
            if (jk < n_tiles) copy_tile(jk, 0, k_s + (jk % kStages) * kKBytes);
            if (jv >= 0) copy_tile(jv, 1, v_s + (jv % kStages) * kVBytes);
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            ++committed;
            if (committed - published >= kInFlight) {
                asm volatile("cp.async.wait_group %0;\n" ::"n"(kInFlight - 1) : "memory");
                publish(published++);
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");   // nothing in flight when this warp leaves
        while (!stop && published < committed) publish(published++);
    } else if (warp >= 4) {
        // -------------------------------------------------------------------- softmax, one row per thread
        const int x = (warp - 4) >> 2, quad = warp & 3, r = quad * 32 + lane;
        const QTile t = x ? qt[1] : qt[0];
        const int pos = t.first_pos + r;
        const int min_key = window > 0 ? pos - window + 1 : 0;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const uint32_t tmem_sx = tmem + lane_sel + x * 128, tmem_ox = tmem + lane_sel + 256 + x * 128;
        uint64_t* const o_full = &bars->o_full[x];
        float m_ref = -INFINITY, l_run = 0.0f;
        bool alive = t.n > 0 && !*aborted;
        for (int j = 0; j < t.n && alive; ++j) {
            const uint32_t t_s = tmem_sx + (j & 1) * kBN;
            if (!mbar_wait(&bars->s_full[x][j & 1], (j >> 1) & 1)) {
                atomicExch(error_word, 10);
                *aborted = 1;
            }
            if (__any_sync(0xffffffffu, *aborted != 0)) { alive = false; break; }     // a warp leaves as one
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            uint32_t sv[kBN];
            tmem_ld32(t_s, *reinterpret_cast<uint32_t(*)[32]>(sv));
            tmem_ld32(t_s + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
            tmem_ld_wait();
            const int key0 = (t.kt_first + j) * kBN;
            // only tiles on the diagonal or at the window's far edge hold keys some row may not see
            if (key0 + kBN - 1 > t.first_pos || (window > 0 && key0 < t.last_pos - window + 1)) {
#pragma unroll
                for (int i = 0; i < kBN; ++i) {
                    const int key = key0 + i;
                    if (key > pos || key < min_key) sv[i] = 0xff800000u;      // -inf
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < kBN; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(sv[i]));
            const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;
            // raise the reference maximum only when this tile is far above it
            const bool raise = tile_max > m_ref + kRaise;
            float factor = 1.0f;
            if (raise) {
                factor = ex2(m_ref - tile_max);             // 0 for the first keys a row sees
                m_ref = tile_max;
                l_run *= factor;
            }
            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                // O holds the tiles before this one: wait for PV(j-1), then scale it down.  (S(j) was
                // issued after PV(j-2) completed and PV(j) waits for this warp, so o_full is in
                // phase j-1 or j: the parity tells them apart.)
                if (!mbar_wait(o_full, (j - 1) & 1)) {
                    atomicExch(error_word, 11);
                    *aborted = 1;
                }
                if (__any_sync(0xffffffffu, *aborted != 0)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                for (int c = 0; c < kHD; c += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem_ox + c, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tmem_st32(tmem_ox + c, o);
                }
                tmem_st_wait();
            }
            const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t pw[kBN / 2];
#pragma unroll
            for (int i = 0; i < kBN; i += 2) {
                const float a = ex2(fmaf(__uint_as_float(sv[i]), scale_log2e, -m_use));
                const float b = ex2(fmaf(__uint_as_float(sv[i + 1]), scale_log2e, -m_use));
                sum[(i >> 1) & 3] += a + b;
                pw[i >> 1] = pack2(a, b);
            }
            l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            tmem_st32(t_s, pw);                              // P over the S it came from
            tmem_st_wait();
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_full[x][j & 1]);
        }
        if (alive) {
            if (!mbar_wait(&bars->o_done[x], 0)) {
                atomicExch(error_word, 12);
                *aborted = 1;
            }
        }
        // ---- result: through shared memory (this query tile is no longer needed) for whole-line stores
        if (t.n > 0) {
            if (x == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
            else asm volatile("bar.sync 2, 128;\n" ::: "memory");
        }
        const bool finish = alive && !__any_sync(0xffffffffu, *aborted != 0);
        if (finish && splits > 1) {
            // ---- one of several runs of keys: O as it stands, its reference maximum and its sum
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const size_t index = part_index(t, r);
#pragma unroll 1
            for (int c = 0; c < kHD; c += 32) {
                uint32_t o[32];
                tmem_ld32(tmem_ox + c, o);
                tmem_ld_wait();
                if (r < t.rows) {
                    uint4* dst = reinterpret_cast<uint4*>(part_o + index * kHD + c);
#pragma unroll
                    for (int e = 0; e < 8; ++e) dst[e] = make_uint4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
                }
            }
            if (r < t.rows) {
                part_ml[index * 2] = m_ref;
                part_ml[index * 2 + 1] = l_run;
            }
        } else if (finish) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = 1.0f / l_run;
            const uint32_t stage = q_s + x * kQBytes, stage_row = stage + r * 256;
#pragma unroll 1
            for (int c = 0; c < kHD; c += 32) {
                uint32_t o[32];
                tmem_ld32(tmem_ox + c, o);
                tmem_ld_wait();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        w[e] = pack2(__uint_as_float(o[q4 * 8 + 2 * e]) * inv, __uint_as_float(o[q4 * 8 + 2 * e + 1]) * inv);
                    const int chunk = c / 8 + q4;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(stage_row + ((chunk ^ (r & 15)) << 4)),
                                 "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                                 : "memory");
                }
            }
            __syncwarp();
            // a warp stores its 32 rows, two rows (2 x 256 bytes) per instruction
#pragma unroll 1
            for (int i = 0; i < 16; ++i) {
                const int rr = quad * 32 + i * 2 + (lane >> 4), c = lane & 15;
                if (rr < t.rows) {
                    uint4 val;
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                                 : "r"(stage + rr * 256 + ((c ^ (rr & 15)) << 4)));
                    *reinterpret_cast<uint4*>(out + ((size_t)(start + t.q_off + rr) * q_heads + t.head) * kHD + c * 8) = val;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// out[row, head, :] = sum_z O_z 2^(m_z - M) / sum_z l_z 2^(m_z - M) over the runs of keys, in
// index order; a run that held no key for the row has m = -inf and is passed over.  A block
// takes kCombineRows rows of one entry of the tile list and one head.
constexpr int kCombineRows = 8;
__global__ void paged_attention_prefill_combine_kernel(const float* part_o, const float* part_ml,
                                                       const int* __restrict__ seg_info,
                                                       const int* __restrict__ tiles, int rows_per_tile,
                                                       int q_heads, int splits, bf16* __restrict__ out) {
    const int seg = tiles[2 * blockIdx.x], q_off = tiles[2 * blockIdx.x + 1], head = blockIdx.y, d = threadIdx.x;
    const int start = seg_info[4 * seg + 1], len = seg_info[4 * seg + 2];
    for (int i = 0; i < kCombineRows; ++i) {
        const int r = q_off + blockIdx.z * kCombineRows + i;
        if (r >= len || r >= q_off + rows_per_tile) return;
        const size_t base = ((size_t)(start + r) * q_heads + head) * splits;
        float mm = -INFINITY;
        for (int z = 0; z < splits; ++z) mm = fmaxf(mm, part_ml[(base + z) * 2]);
        float total = 0.0f, acc = 0.0f;
        for (int z = 0; z < splits; ++z) {
            const float mz = part_ml[(base + z) * 2];
            if (mz == -INFINITY) continue;
            const float f = exp2f(mz - mm);
            total += part_ml[(base + z) * 2 + 1] * f;
            acc += part_o[(base + z) * kHD + d] * f;
        }
        out[((size_t)(start + r) * q_heads + head) * kHD + d] = __float2bfloat16_rn(acc / total);
    }
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

// [rows, cols] bfloat16 row-major, boxes of box_rows x 64 columns, 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace pftc
}  // namespace tllm

using namespace tllm;

// Query rows per block of the tile list: 128 where two heads of a key/value head share a block
// (an even group), else 256 (two blocks of positions of one head).
extern "C" int tllm_paged_attention_prefill_tc_rows(int q_heads, int kv_heads) {
    return (kv_heads > 0 && q_heads % kv_heads == 0 && (q_heads / kv_heads) % 2 == 0) ? 128 : 256;
}

// tiles: int[n_tiles][2] = segment, offset of the block's first query row; the offsets are the
// multiples of tllm_paged_attention_prefill_tc_rows() below the segment's length.
// q [tokens, q_heads * 128], cache [num_pages, 2, kv_heads, page_size, 128], both bfloat16.
// splits > 1: the keys of every block go to that many blocks in equal runs (for steps with few
// query rows and many keys, which would leave most of the GPU idle), their partial results to
// part_o float[tokens * q_heads * splits * 128] and part_ml float[tokens * q_heads * splits * 2],
// and a second kernel combines them.
extern "C" int tllm_paged_attention_prefill_tc(
    const void* q, int tokens, const void* cache, int num_pages, const int* seg_info, const int* tiles, int n_tiles,
    const int* block_table, int max_pages, int page_size, int q_heads, int kv_heads, int head_dim, int window,
    float scale, void* out, int splits, float* part_o, float* part_ml, int* error_word, cudaStream_t stream) {
    TLLM_REQUIRE(head_dim == 128, "paged_attention_prefill_tc: head_dim %d is not 128", head_dim);
    TLLM_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads <= 65535,
                 "paged_attention_prefill_tc: %d query heads over %d key/value heads", q_heads, kv_heads);
    TLLM_REQUIRE(page_size > 0 && page_size % 16 == 0, "paged_attention_prefill_tc: page size %d is no multiple of 16",
                 page_size);
    TLLM_REQUIRE(error_word != nullptr && n_tiles >= 0 && n_tiles <= 65535 && tokens > 0,
                 "paged_attention_prefill_tc: bad arguments (at most 65535 blocks of query rows)");
    TLLM_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || (part_o != nullptr && part_ml != nullptr)),
                 "paged_attention_prefill_tc: %d splits (1 to 64; more than one needs scratch)", splits);
    const long long kv_rows = (long long)num_pages * 2 * kv_heads * page_size;
    TLLM_REQUIRE(kv_rows < (1ll << 31), "paged_attention_prefill_tc: a cache of %lld rows exceeds the kernel's 32-bit row index",
                 kv_rows);
    if (n_tiles == 0) return 0;
    TLLM_REQUIRE((reinterpret_cast<uintptr_t>(cache) & 15u) == 0 && (reinterpret_cast<uintptr_t>(q) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 15u) == 0 && (reinterpret_cast<uintptr_t>(part_o) & 15u) == 0,
                 "paged_attention_prefill_tc: pointers must be 16-byte aligned");
    CUtensorMap mq;
    TLLM_REQUIRE(pftc::make_map(&mq, q, tokens, (long long)q_heads * 128, 128),
                 "paged_attention_prefill_tc: cuTensorMapEncodeTiled failed or is not available");
    static OncePerDevice configured;
    if (configured.first()) {
        cudaError_t e = cudaFuncSetAttribute(pftc::paged_attention_prefill_tc_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, pftc::kSmemBytes);
        if (e != cudaSuccess) { set_error("paged_attention_prefill_tc: %s", cudaGetErrorString(e)); return (int)e; }
        configured.done();
    }
    const int rows_per_tile = tllm_paged_attention_prefill_tc_rows(q_heads, kv_heads);
    const int pair_heads = rows_per_tile == 128;
    pftc::paged_attention_prefill_tc_kernel<<<dim3(pair_heads ? q_heads / 2 : q_heads, n_tiles, splits), pftc::kThreads,
                                              pftc::kSmemBytes, stream>>>(
        mq, (const bf16*)cache, seg_info, tiles, block_table, max_pages, page_size, q_heads, kv_heads, window,
        scale * 1.4426950408889634f, pair_heads, (bf16*)out, splits, part_o, part_ml, error_word);
    int rc = finish_launch("paged_attention_prefill_tc");
    if (rc != 0 || splits == 1) return rc;
    pftc::paged_attention_prefill_combine_kernel<<<dim3(n_tiles, q_heads, rows_per_tile / pftc::kCombineRows), 128, 0, stream>>>(
        part_o, part_ml, seg_info, tiles, rows_per_tile, q_heads, splits, (bf16*)out);
    return finish_launch("paged_attention_prefill_combine");
}
