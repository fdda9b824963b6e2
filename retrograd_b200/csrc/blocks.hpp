// GGUF tensor storage formats this backend reads, and host-side scalar helpers.
//
// Block geometry follows the reference's in-tree format table
// (crates/rir-core/src/quant_table.rs:322-360,420-440; decoders in
// crates/rir-core/src/quant.rs:223-417):
//   Q8_0   32 elements / 34 B : f16 d | 32 x i8
//   Q4_K  256 elements / 144 B: f16 d | f16 dmin | 12 B packed 6-bit scales+mins | 128 B nibbles
//   MXFP4  32 elements / 17 B : E8M0 exponent byte | 16 B nibbles (doubled E2M1 table)
#pragma once

#include <cstdint>
#include <cstddef>
#include <cstring>
#include <cmath>

namespace rb200 {

enum GgmlType : uint32_t {
    GGML_F32 = 0,
    GGML_F16 = 1,
    GGML_Q8_0 = 8,
    GGML_Q4_K = 12,
    GGML_BF16 = 30,
    GGML_MXFP4 = 39,
};

struct BlockGeom {
    uint32_t elems;
    uint32_t bytes;
};

inline bool block_geom(uint32_t type, BlockGeom & out) {
    switch (type) {
        case GGML_F32:   out = {1, 4};     return true;
        case GGML_F16:   out = {1, 2};     return true;
        case GGML_BF16:  out = {1, 2};     return true;
        case GGML_Q8_0:  out = {32, 34};   return true;
        case GGML_Q4_K:  out = {256, 144}; return true;
        case GGML_MXFP4: out = {32, 17};   return true;
        default: return false;
    }
}

inline const char * type_name(uint32_t type) {
    switch (type) {
        case GGML_F32: return "f32";
        case GGML_F16: return "f16";
        case GGML_BF16: return "bf16";
        case GGML_Q8_0: return "q8_0";
        case GGML_Q4_K: return "q4_K";
        case GGML_MXFP4: return "mxfp4";
        default: return "unsupported";
    }
}

// Bytes of `n` elements stored as `type` (n must be a whole number of blocks).
inline size_t row_bytes(uint32_t type, size_t n) {
    BlockGeom g{};
    if (!block_geom(type, g) || n % g.elems != 0) return 0;
    return n / g.elems * g.bytes;
}

// IEEE binary16 <-> binary32, exact, host side.
inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31;
    const uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = 0;
            while (!(man & 0x400)) { man <<= 1; ++e; }
            man &= 0x3ff;
            bits = sign | ((uint32_t)(113 - e) << 23) | (man << 13);
        }
    } else if (exp == 0x1f) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// Round-to-nearest-even, overflow to infinity.
inline uint16_t float_to_half(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) {
        return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
    }
    if (x >= 0x477ff000u) {
        return (uint16_t)(sign | 0x7c00u);
    }
    if (x < 0x38800000u) {
        // subnormal half (or zero)
        if (x < 0x33000000u) return (uint16_t)sign;
        const int shift = 126 - (int)(x >> 23);   // 14..24
        uint32_t man = (x & 0x7fffffu) | 0x800000u;
        const uint32_t rem_mask = (1u << shift) - 1;
        const uint32_t rem = man & rem_mask;
        const uint32_t half = 1u << (shift - 1);
        man >>= shift;
        if (rem > half || (rem == half && (man & 1))) ++man;
        return (uint16_t)(sign | man);
    }
    uint32_t man = x & 0x7fffffu;
    uint32_t exp = (x >> 23) - 112;
    uint32_t out = (exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (out & 1))) ++out;
    return (uint16_t)(sign | out);
}

inline float bf16_to_float(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// The E8M0 exponent byte scaled by 1/2, the convention the doubled E2M1 table expects.
inline float e8m0_half_to_float(uint8_t x) {
    uint32_t bits = x == 0 ? 0x00200000u : x == 1 ? 0x00400000u : ((uint32_t)x - 1) << 23;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// The 6-bit (scale, min) pair of sub-block j from the 12 packed bytes of a Q4_K block.
inline void q4k_scale_min(int j, const uint8_t * q, uint8_t & sc, uint8_t & mn) {
    if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

} // namespace rb200
