// Device helpers that write an activation in the form the exact tensor-core GEMMs read: the two-term
// f16 split x = hi + lo and, per 32-column sub-block, the sum of x as hi + lo.
#pragma once

#include "kernels.cuh"

namespace rb200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Writes v as hi + lo and, once per warp, the sub-block sum of v as hi + lo. Every lane of the
// warp must call it, with 32 consecutive columns starting at a multiple of 32.
__device__ __forceinline__ void emit_split(const SplitAct & s, size_t row, int col, float v) {
    const __half hi = __float2half_rn(v);
    const size_t at = row * s.ld + col;
    s.hi[at] = hi;
    s.lo[at] = __float2half_rn(v - __half2float(hi));
    const float sum = warp_sum(v);
    if ((threadIdx.x & 31) == 0) {
        const __half sh = __float2half_rn(sum);
        const size_t sat = row * (s.ld >> 5) + (col >> 5);
        s.sum_hi[sat] = sh;
        s.sum_lo[sat] = __float2half_rn(sum - __half2float(sh));
    }
}

// Four consecutive columns per thread (col % 4 == 0): eight neighbouring lanes cover one 32-column
// sub-block. Every lane of the warp must call it; `active` masks the stores of lanes past the row.
__device__ __forceinline__ void emit_split4(const SplitAct & s, size_t row, int col, float4 v, bool active) {
    const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(v.x - f01.x, v.y - f01.y), l23 = __floats2half2_rn(v.z - f23.x, v.w - f23.y);
    float sum = active ? (v.x + v.y) + (v.z + v.w) : 0.f;
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if (!active) return;
    const size_t at = row * s.ld + col;
    *reinterpret_cast<uint2 *>(s.hi + at) = make_uint2(*reinterpret_cast<const uint32_t *>(&h01), *reinterpret_cast<const uint32_t *>(&h23));
    *reinterpret_cast<uint2 *>(s.lo + at) = make_uint2(*reinterpret_cast<const uint32_t *>(&l01), *reinterpret_cast<const uint32_t *>(&l23));
    if ((threadIdx.x & 7) == 0) {
        const __half sh = __float2half_rn(sum);
        const size_t sat = row * (s.ld >> 5) + (col >> 5);
        s.sum_hi[sat] = sh;
        s.sum_lo[sat] = __float2half_rn(sum - __half2float(sh));
    }
}

} // namespace rb200
