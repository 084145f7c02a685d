// Warp-level tensor-core building blocks shared by the bfloat16 attention kernels:
// mma.sync m16n8k16 (bf16 x bf16 -> f32), ldmatrix, cp.async and the shared-memory
// swizzle that keeps ldmatrix free of bank conflicts.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace tllm {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// D[16x8] += A[16x16] * B[16x8]; A row-major fragments, B column fragments.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4],
                                               const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// 16-byte asynchronous copy global -> shared; `valid == false` writes zeros instead.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile of rows of HD bf16 (HD * 2 bytes per row, HD a multiple of 64) in shared memory.
// The 16-byte chunk c of row r lives at chunk c ^ (r & 7): eight rows read at the same
// logical chunk (one ldmatrix phase) fall into eight different bank groups.
template <int HD>
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) {
    return (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

}  // namespace tllm
