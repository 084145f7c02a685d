// Shared device helpers of the sm_100a kernels: storage-type conversion, warp and
// block reductions, error reporting of the C entry points.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace tllm {

// Storage types are selected at run time by these codes in every C entry point.
enum DType : int { kF32 = 0, kBF16 = 1 };

using bf16 = __nv_bfloat16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  Every thread
// gets the result.  The order of the additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    return warp_sum(r);
}

// Programmatic dependent launch.  A kernel launched with `launch_pdl` may be scheduled while
// the kernel before it in the stream is still running; it must execute TLLM_PDL_ENTER()
// (or TLLM_PDL_WAIT() after a prologue that touches nothing an earlier kernel writes or
// reads) before its first access to memory that earlier kernels produce or still read.
// Kernels that are a few microseconds long, as in a decode step, then no longer pay their
// launch and ramp-up one after the other.
#define TLLM_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;\n" ::)
#define TLLM_PDL_WAIT() asm volatile("griddepcontrol.wait;\n" ::: "memory")
#define TLLM_PDL_ENTER() \
    do {                 \
        TLLM_PDL_TRIGGER(); \
        TLLM_PDL_WAIT();    \
    } while (0)

// Whether `launch_pdl` really asks for the early start, by the class of the kernel.  Measured on
// a decode step of a Qwen3-8B-sized model (4.16 ms): early starts pay for the kernels that have
// something to fetch before they wait (the weight-streaming product, which always asks); for the
// short kernels between them an ordinary launch is as fast or faster (norm 4.17 ms, q/k 4.17,
// SwiGLU 4.22, attention 4.22, combine 4.24), and when several classes start early at once whole
// chains of products are resident and fetching long before their turn (norm + q/k + SwiGLU +
// combine: 4.93 ms).  A later measurement, three runs each way on one GPU, found the residual add + norm
// to gain a little after all (batch 8: 4.086 to 4.052 ms, batch 1: 3.33 to 3.32, batch 64: 9.59 to
// 9.58), so that class is on by default and the others are off; the environment variable TLLM_PDL
// holds the sum of the classes to switch on instead, for measurements.  All kernels still let their
// successor start early.
enum PdlClass { kPdlNorm = 1, kPdlQk = 2, kPdlSwiglu = 4, kPdlAttention = 8, kPdlCombine = 16, kPdlOther = 32, kPdlAlways = 1 << 20 };

inline bool pdl_enabled(int cls) {
    static const int mask = [] { const char* v = getenv("TLLM_PDL"); return v != nullptr ? atoi(v) : (int)kPdlNorm; }();
    return cls == kPdlAlways || (mask & cls) != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(int cls, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(cls) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Set-up that a launcher does once per device (a function attribute belongs to the device that was
// current when it was set): `OncePerDevice flag;` as a function-local static, then
// `if (flag.first()) { ...; flag.done(); }`.  first() is false for a device index it cannot tell or
// hold, so that the set-up is then simply repeated at every call.
struct OncePerDevice {
    static constexpr int kMax = 64;
    bool seen[kMax] = {};
    int device = -1;
    bool first() {
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMax) { device = -1; return true; }
        return !seen[device];
    }
    void done() { if (device >= 0) seen[device] = true; }
};

// Multiprocessors of the current device (0 if that cannot be told), looked up once per device.
inline int sm_count_cached() {
    static int count[OncePerDevice::kMax] = {};
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= OncePerDevice::kMax) return 0;
    if (count[device] == 0 &&
        cudaDeviceGetAttribute(&count[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        count[device] = 0;
    return count[device];
}

// Host side: the last error text of this thread's most recent failing entry point.
void set_error(const char* fmt, ...);

// Result of an entry point: 0 on success, a cudaError_t (> 0) from the launch, or
// -1 for an argument the kernel refuses (text in tllm_last_error()).
int finish_launch(const char* what);

#define TLLM_REQUIRE(cond, ...)                 \
    do {                                        \
        if (!(cond)) {                          \
            ::tllm::set_error(__VA_ARGS__);     \
            return -1;                          \
        }                                       \
    } while (0)

}  // namespace tllm
