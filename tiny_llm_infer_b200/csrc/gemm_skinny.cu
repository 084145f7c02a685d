// y[M, N] = x[M, K] . W[N, K]^T for a handful of rows (M <= 32), bfloat16 in, float32
// accumulation: the product of a decode step, where every weight is read once and the time
// is the time HBM needs to deliver the weights.
//
// The reference has a one-row kernel for this (matmul_fp16_gemv_kernel,
// kernels/src/matmul_kernel_cuda.cu:17-32: one block per output, scalar half loads) and
// falls back to the library for two rows and more.  Here a block owns 16 rows of W and its
// eight warps split K.  A lane reads 16 contiguous bytes of a weight row at a time with a
// streaming load and feeds them to mma.sync m16n8k16 with W as the A operand (16 weight
// rows) and the activations as the B operand (8 tokens per tile): because a sum does not
// care about the order of its terms, the eight neighbouring k's of a lane can stand for the
// k-columns the fragment layout assigns to it, in two mma steps, provided the activations
// are permuted the same way, which a 16-byte load of x does by itself.  No shared memory,
// no shuffles on the way in; loads of the next k-blocks are in flight while the current
// ones are multiplied; the warps' partial sums meet in shared memory at the end and are
// added in warp order.
//
// The kernel is launched with programmatic dependent launch: it may start while the kernel
// before it in the stream is still draining, fetches its first weights (which depend on
// nothing), and only then waits for that kernel's results (griddepcontrol.wait) before it
// touches the activations or writes anything.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace tllm {

constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyUnroll = 2;      // k-blocks of 32 per pipeline stage

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// The activations were written by the kernel this one may have started beside: they are
// read with an ordinary (coherent) load after the wait, never through the read-only path,
// whose contract (data constant for the kernel's lifetime) an early start would break.
__device__ __forceinline__ uint4 ld_coherent(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

template <int NT>
struct SkinnyStage {
    uint4 a_lo[kSkinnyUnroll], a_hi[kSkinnyUnroll], b[kSkinnyUnroll][NT];
};

// The warps' partial sums, left in `red`, are added in warp order and written.  Kept out of line:
// inlined, the SwiGLU form costs the kernel ten registers more than the plain one (88 instead of
// 78) and with them the third block per SM (the gate/up product of Qwen3-8B sizes: 42.5 us at two
// blocks per SM, 35.1 at three, as the plain product of the same rows).
template <int NT, typename TOut, bool SWIGLU>
__device__ __noinline__ void skinny_epilogue(float (*red)[16][NT * 8 + 1], TOut* y, int M, int N, int r0) {
    constexpr int kRows = SWIGLU ? 8 : 16;                   // output columns of the block
    for (int idx = threadIdx.x; idx < kRows * NT * 8; idx += blockDim.x) {
        const int row = idx % kRows, tok = idx / kRows;
        if (tok < M && r0 + row < N) {
            float s = 0.0f;
#pragma unroll
            for (int ww = 0; ww < kSkinnyWarps; ++ww) s += red[ww][row][tok];
            if (SWIGLU) {
                float up = 0.0f;
#pragma unroll
                for (int ww = 0; ww < kSkinnyWarps; ++ww) up += red[ww][row + 8][tok];
                s = s / (1.0f + expf(-s)) * up;
            }
            y[(size_t)tok * N + r0 + row] = from_f32<TOut>(s);
        }
    }
}

// SWIGLU: w holds N gate rows and N up rows interleaved by eight (eight gate rows, their eight up
// rows, and so on); the block's 16-row tile is eight gate rows as its upper half and the up rows
// that belong to them as its lower half, so that a gate sum and its up sum meet in one thread's
// accumulator; it writes silu(gate) * up: y is [M, N].  The grid, the bytes per block, the memory
// pattern and the registers are those of the plain product of the 2 N rows.
template <int NT, typename TOut, bool SWIGLU, int STAGES>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
skinny_gemm_kernel(const bf16* x, const bf16* __restrict__ w, TOut* y, int M, int N, int K) {
    __shared__ float red[kSkinnyWarps][16][NT * 8 + 1];
    asm volatile("griddepcontrol.launch_dependents;\n" ::);
    const int r0 = blockIdx.x * (SWIGLU ? 8 : 16);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, c = lane & 3, rq = lane >> 2;
    // first rows of the tile's halves in w (SWIGLU: r0 counts outputs, and N % 8 == 0)
    const size_t lo_row = !SWIGLU ? min(r0 + rq, N - 1) : 2 * r0 + rq;
    const size_t hi_row = !SWIGLU ? min(r0 + rq + 8, N - 1) : lo_row + 8;
    const bf16* w_lo = w + lo_row * K;
    const bf16* w_hi = w + hi_row * K;
    const bf16* xr[NT];
    bool xv[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int tok = nt * 8 + rq;
        xv[nt] = tok < M;
        xr[nt] = x + (size_t)(xv[nt] ? tok : 0) * K;
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;

    const int kblocks = (K + 31) >> 5;                       // 32 k per block: 8 per lane of a quad
    const int per_warp = (kblocks + kSkinnyWarps - 1) / kSkinnyWarps;
    const int kb0 = warp * per_warp, kb1 = min(kblocks, kb0 + per_warp);
    const uint4 zero = make_uint4(0, 0, 0, 0);

    auto load_w = [&](SkinnyStage<NT>& s, int kb) {
#pragma unroll
        for (int u = 0; u < kSkinnyUnroll; ++u) {
            const int k = (kb + u) * 32 + c * 8;
            const bool ok = kb + u < kb1 && k < K;
            s.a_lo[u] = ok ? ld_stream(w_lo + k) : zero;
            s.a_hi[u] = ok ? ld_stream(w_hi + k) : zero;
        }
    };
    auto load_x = [&](SkinnyStage<NT>& s, int kb) {
#pragma unroll
        for (int u = 0; u < kSkinnyUnroll; ++u) {
            const int k = (kb + u) * 32 + c * 8;
            const bool ok = kb + u < kb1 && k < K;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                s.b[u][nt] = (ok && xv[nt]) ? ld_coherent(xr[nt] + k) : zero;
        }
    };
    auto multiply = [&](const SkinnyStage<NT>& s) {
#pragma unroll
        for (int u = 0; u < kSkinnyUnroll; ++u) {
            const uint32_t a1[4] = {s.a_lo[u].x, s.a_hi[u].x, s.a_lo[u].y, s.a_hi[u].y};
            const uint32_t a2[4] = {s.a_lo[u].z, s.a_hi[u].z, s.a_lo[u].w, s.a_hi[u].w};
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t b1[2] = {s.b[u][nt].x, s.b[u][nt].y}, b2[2] = {s.b[u][nt].z, s.b[u][nt].w};
                mma_bf16_16816(acc[nt], a1, b1);
                mma_bf16_16816(acc[nt], a2, b2);
            }
        }
    };

    // STAGES - 1 stages are on their way while one is multiplied
    SkinnyStage<NT> st[STAGES];
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) load_w(st[i], kb0 + i * kSkinnyUnroll);   // weights depend on no earlier kernel
    asm volatile("griddepcontrol.wait;\n" ::: "memory");     // from here on x may be read, y written
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) load_x(st[i], kb0 + i * kSkinnyUnroll);
    for (int kb = kb0; kb < kb1; kb += STAGES * kSkinnyUnroll) {
#pragma unroll
        for (int i = 0; i < STAGES; ++i) {
            constexpr int kLast = STAGES - 1;
            load_w(st[(i + kLast) % STAGES], kb + (i + kLast) * kSkinnyUnroll);
            load_x(st[(i + kLast) % STAGES], kb + (i + kLast) * kSkinnyUnroll);
            multiply(st[i]);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][rq][nt * 8 + c * 2] = acc[nt][0];
        red[warp][rq][nt * 8 + c * 2 + 1] = acc[nt][1];
        red[warp][rq + 8][nt * 8 + c * 2] = acc[nt][2];
        red[warp][rq + 8][nt * 8 + c * 2 + 1] = acc[nt][3];
    }
    __syncthreads();
    skinny_epilogue<NT, TOut, SWIGLU>(red, y, M, N, r0);
}

template <int NT, typename TOut, bool SWIGLU, int STAGES = 3>
static int launch_skinny(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SWIGLU ? (N + 7) / 8 : (N + 15) / 16);
    cfg.blockDim = dim3(kSkinnyWarps * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_gemm_kernel<NT, TOut, SWIGLU, STAGES>, (const bf16*)x, (const bf16*)w,
                                       (TOut*)y, M, N, K);
    if (e != cudaSuccess) {
        set_error("gemm_skinny: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return finish_launch("gemm_skinny");
}

}  // namespace tllm

using namespace tllm;

// out_dtype: storage type of y (bfloat16 or float32).  K must be a multiple of 8 and x, w
// 16-byte aligned; M at most 32.
extern "C" int tllm_gemm_skinny(const void* x, const void* w, void* y, int out_dtype, int M, int N, int K,
                                cudaStream_t stream) {
    TLLM_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_skinny: bad sizes");
    TLLM_REQUIRE(M <= 32, "gemm_skinny: %d rows exceed 32", M);
    TLLM_REQUIRE(K % 8 == 0, "gemm_skinny: K = %d is no multiple of 8", K);
    TLLM_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15u) == 0,
                 "gemm_skinny: operands must be 16-byte aligned");
    TLLM_REQUIRE(out_dtype == kBF16 || out_dtype == kF32, "gemm_skinny: unknown output dtype");
    if (M == 0) return 0;
    if (out_dtype == kBF16) {
        // A grid that leaves room on the GPU takes its registers for a deeper pipeline instead (the
        // kernel of three stages holds three blocks per SM, of four two, of six one): alone, the o and
        // down products of Qwen3-8B sizes (256 blocks) 8.4 to 7.9 and 20.0 to 18.6 us with four stages,
        // those of Qwen3-0.6B sizes (64 blocks) 3.8 to 2.7 and 4.5 to 3.5 us with six.  With more blocks
        // than places (320 blocks of Qwen3-32B sizes on 296) four stages take 14 us instead of 10, and a
        // warp with four k-blocks or fewer to walk (K = 1024) has nothing to put into them.
        if (M <= 8) {
            const int sms = sm_count_cached();
            const long long blocks = ((long long)N + 15) / 16;
            if (blocks <= sms && K >= 2048) return launch_skinny<1, bf16, false, 6>(x, w, y, M, N, K, stream);
            if (blocks <= 2ll * sms && K >= 4096) return launch_skinny<1, bf16, false, 4>(x, w, y, M, N, K, stream);
        }
        if (M <= 8) return launch_skinny<1, bf16, false>(x, w, y, M, N, K, stream);
        if (M <= 16) return launch_skinny<2, bf16, false>(x, w, y, M, N, K, stream);
        return launch_skinny<4, bf16, false>(x, w, y, M, N, K, stream);
    }
    if (M <= 8) return launch_skinny<1, float, false>(x, w, y, M, N, K, stream);
    if (M <= 16) return launch_skinny<2, float, false>(x, w, y, M, N, K, stream);
    return launch_skinny<4, float, false>(x, w, y, M, N, K, stream);
}

// y[M, N] = silu(x . gate^T) * (x . up^T) for w of 2 N rows, gate and up interleaved by eight
// (eight gate rows, their eight up rows, ...), bfloat16 out, M <= 16.
extern "C" int tllm_gemm_skinny_swiglu(const void* x, const void* w, void* y, int M, int N, int K,
                                       cudaStream_t stream) {
    TLLM_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_skinny_swiglu: bad sizes");
    TLLM_REQUIRE(M <= 16, "gemm_skinny_swiglu: %d rows exceed 16", M);
    TLLM_REQUIRE(N % 8 == 0, "gemm_skinny_swiglu: N = %d is no multiple of 8", N);
    TLLM_REQUIRE(K % 8 == 0, "gemm_skinny_swiglu: K = %d is no multiple of 8", K);
    TLLM_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15u) == 0,
                 "gemm_skinny_swiglu: operands must be 16-byte aligned");
    if (M == 0) return 0;
    if (M <= 8) return launch_skinny<1, bf16, true>(x, w, y, M, N, K, stream);
    return launch_skinny<2, bf16, true>(x, w, y, M, N, K, stream);
}
