// Warp-level tensor-core and asynchronous-copy primitives shared by the bfloat16
// attention kernels: cp.async (16-byte, zero-filling), ldmatrix, and the
// m16n8k16 bf16 MMA with float accumulation.
//
// Fragment layouts (lane = threadIdx.x % 32, g = lane / 4, t = lane % 4):
//   A 16x16 row-major, 4 regs: (row g, cols 2t..2t+1), (row g+8, same), (row g, cols
//     2t+8..2t+9), (row g+8, same)
//   B 16x8 "col" (k x n), 2 regs: (k 2t..2t+1, n g), (k 2t+8..2t+9, n g)
//   C 16x8, 4 floats: (row g, cols 2t, 2t+1), (row g+8, cols 2t, 2t+1)
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 16 bytes global -> shared; src_bytes == 0 writes zeros (src must still be a valid address)
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
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

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Position (in elements) of 16-byte chunk `c` of row `row` in a shared tile whose rows
// hold CPR chunks.  Rows of 128 bytes or more are XOR-swizzled so that the eight rows an
// ldmatrix reads fall into different banks.
template <int CPR> __device__ __forceinline__ int tile_off(int row, int c) {
    return row * (CPR * 8) + ((CPR >= 8 ? (c ^ (row & 7)) : c) << 3);
}
