// Shared device helpers of the tensor-core kernels: cp.async, ldmatrix, mma.sync m16n8k16 and
// the 128-byte XOR swizzle of [rows][64 x f16] shared-memory tiles.
#pragma once

#include <cstdint>
#include <cuda_fp16.h>

namespace rb200 {

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The first product of an accumulation chain: d = a b (+ 0), no zeroed accumulator registers needed.
__device__ __forceinline__ void mma_f16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a [rows][128 B] swizzled tile.
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// The 6-bit (scale, min) pair of sub-block j of a Q4_K block whose first 16 bytes are `hdr`
// (hdr.x = d|dmin, hdr.y/z/w = the 12 packed bytes).
__device__ __forceinline__ void q4k_scale_min_regs(const uint4 & hdr, int j, uint32_t & sc, uint32_t & mn) {
    if (j < 4) {
        sc = (hdr.y >> (8 * j)) & 63u;
        mn = (hdr.z >> (8 * j)) & 63u;
    } else {
        const int jj = j - 4;
        const uint32_t lo = (hdr.w >> (8 * jj)) & 0xFFu;
        sc = (lo & 0xFu) | ((((hdr.y >> (8 * jj)) & 0xFFu) >> 6) << 4);
        mn = (lo >> 4) | ((((hdr.z >> (8 * jj)) & 0xFFu) >> 6) << 4);
    }
}

} // namespace rb200
