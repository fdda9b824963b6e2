// Dequant-fused weight GEMM for many tokens per step (prefill chunks, wide decode batches):
//   Y[t][o] = sum_k deq(W)[o][k] * X[t][k]  (+ bias[o]) (+ residual[t][o])
// Weights stay in HBM in their GGUF block layout and are streamed exactly once per CTA column:
// each 128-row x 64-column weight tile is decoded in registers (nibbles -> f16 with the 0x6400
// exponent trick, sub-block scale and min folded in with one half2 FMA) into a 128B-swizzled
// shared-memory tile, activations arrive as f16 through cp.async, and the contraction runs on
// the tensor cores with f32 accumulation (mma.sync m16n8k16; weights are the M operand so a
// small token count wastes nothing). Three stages of shared memory overlap the global loads,
// the decode and the MMAs.
//
// Accuracy: weights and activations are rounded to f16 (11-bit significands) before the
// contraction, which keeps fp32 logits of an 8B-shape model well inside the 1e-2 tolerance; the
// row kernel in kernels.cu is the f32 reference and serves the steps with few tokens.

#include "kernels.cuh"
#include "blocks.hpp"

#include <cuda_fp16.h>

namespace rb200 {

namespace {

constexpr int BM = 128;      // weight rows per CTA
constexpr int BK = 64;       // contraction depth per stage (one 64-element group of a Q4_K block)
constexpr int STAGES = 3;
constexpr int THREADS = 256;

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a [rows][128 B] swizzled tile.
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

struct Q4kFetch {
    uint4 hdr;   // d, dmin, 12 scale bytes
    uint4 q0, q1;
};

// Four nibbles of one word -> four f16 weights in element order: w = dl * q - ml.
__device__ __forceinline__ void nibbles_to_half(uint32_t word, int hi, __half2 dl2, __half2 ml2, uint32_t & out01, uint32_t & out23) {
    const uint32_t v = hi ? (word >> 4) : word;
    uint32_t a = (v & 0x000F000Fu) | 0x64006400u;          // elements 0 and 2 as 1024 + q
    uint32_t b = ((v >> 8) & 0x000F000Fu) | 0x64006400u;   // elements 1 and 3
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
    __half2 ha = __hsub2(*reinterpret_cast<__half2 *>(&a), k1024);
    __half2 hb = __hsub2(*reinterpret_cast<__half2 *>(&b), k1024);
    ha = __hfma2(ha, dl2, ml2);
    hb = __hfma2(hb, dl2, ml2);
    const uint32_t ua = *reinterpret_cast<uint32_t *>(&ha), ub = *reinterpret_cast<uint32_t *>(&hb);
    out01 = __byte_perm(ua, ub, 0x5410);
    out23 = __byte_perm(ua, ub, 0x7632);
}

template <int BN, bool RESIDUAL>
__global__ void __launch_bounds__(THREADS) gemm_q4k_mma_kernel(const uint8_t * __restrict__ W, int n_in, int n_out, int row_bytes,
                                                               const __half * __restrict__ X, int ldx, int T, float * __restrict__ Y, int ldy,
                                                               const float * __restrict__ bias, const float * __restrict__ residual, int ldr) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int A_BYTES = BM * 128;
    constexpr int B_BYTES = BN * 128;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int WN = BN >= 64 ? 2 : 1;              // warps along the token dimension
    constexpr int WM = 8 / WN;                        // warps along the weight-row dimension
    constexpr int WARP_M = BM / WM;                   // 32 or 16
    constexpr int WARP_N = BN / WN;
    constexpr int MI = WARP_M / 16;
    constexpr int NI = WARP_N / 8;
    static_assert(NI % 2 == 0, "token tiles are loaded in pairs");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % WM, wn = warp / WM;
    const int m0 = blockIdx.x * BM, t0 = blockIdx.y * BN;
    const int n_k = n_in / BK;

    // A producer mapping: two threads per weight row, one per 32-element sub-block
    const int a_row = tid >> 1, a_half = tid & 1;
    const bool a_valid = m0 + a_row < n_out;
    const uint8_t * a_base = W + (size_t)(m0 + (a_valid ? a_row : 0)) * row_bytes;

    auto fetch_a = [&](int kt, Q4kFetch & f) {
        if (!a_valid) return;
        const int k0 = kt * BK;
        const uint8_t * blk = a_base + (size_t)(k0 >> 8) * 144;
        f.hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint4 * qs = reinterpret_cast<const uint4 *>(blk + 16 + ((k0 & 255) >> 6) * 32);
        f.q0 = qs[0];
        f.q1 = qs[1];
    };
    auto store_a = [&](int kt, int stage, const Q4kFetch & f) {
        uint8_t * a_s = smem + stage * STAGE_BYTES;
        uint4 out[4];
        if (a_valid) {
            const int j = (((kt * BK) & 255) >> 6) * 2 + a_half;
            // the 12 packed scale bytes live in hdr.y, hdr.z, hdr.w
            uint32_t sc, mn;
            if (j < 4) {
                sc = (f.hdr.y >> (8 * j)) & 63u;
                mn = (f.hdr.z >> (8 * j)) & 63u;
            } else {
                const int jj = j - 4;
                const uint32_t lo = (f.hdr.w >> (8 * jj)) & 0xFFu;
                sc = (lo & 0xFu) | ((((f.hdr.y >> (8 * jj)) & 0xFFu) >> 6) << 4);
                mn = (lo >> 4) | ((((f.hdr.z >> (8 * jj)) & 0xFFu) >> 6) << 4);
            }
            const __half2 dd = *reinterpret_cast<const __half2 *>(&f.hdr.x);
            const float dl = __low2float(dd) * (float)sc, ml = __high2float(dd) * (float)mn;
            const __half2 dl2 = __float2half2_rn(dl), ml2 = __float2half2_rn(-ml);
            nibbles_to_half(f.q0.x, a_half, dl2, ml2, out[0].x, out[0].y);
            nibbles_to_half(f.q0.y, a_half, dl2, ml2, out[0].z, out[0].w);
            nibbles_to_half(f.q0.z, a_half, dl2, ml2, out[1].x, out[1].y);
            nibbles_to_half(f.q0.w, a_half, dl2, ml2, out[1].z, out[1].w);
            nibbles_to_half(f.q1.x, a_half, dl2, ml2, out[2].x, out[2].y);
            nibbles_to_half(f.q1.y, a_half, dl2, ml2, out[2].z, out[2].w);
            nibbles_to_half(f.q1.z, a_half, dl2, ml2, out[3].x, out[3].y);
            nibbles_to_half(f.q1.w, a_half, dl2, ml2, out[3].z, out[3].w);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4 *>(a_s + swz(a_row, a_half * 4 + c)) = out[c];
    };
    auto load_b = [&](int kt, int stage) {
        const uint32_t b_s = smem_u32(smem + stage * STAGE_BYTES + A_BYTES);
        const int k0 = kt * BK;
#pragma unroll
        for (int i = 0; i < (BN * 8 + THREADS - 1) / THREADS; ++i) {
            const int idx = tid + i * THREADS;
            if (BN * 8 < THREADS && idx >= BN * 8) break;
            const int r = idx >> 3, c = idx & 7;
            const int t = t0 + r;
            const __half * src = X + (size_t)(t < T ? t : 0) * ldx + k0 + c * 8;
            cp_async16(b_s + swz(r, c), src, t < T ? 16 : 0);
        }
    };

    float acc[MI][NI][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < NI; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mi][ni][e] = 0.f;

    Q4kFetch fetch;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_k) {
            load_b(s, s);
            fetch_a(s, fetch);
            store_a(s, s, fetch);
        }
        cp_async_commit();
    }

    for (int kt = 0; kt < n_k; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        const int next = kt + STAGES - 1;
        if (next < n_k) {
            load_b(next, next % STAGES);
            fetch_a(next, fetch);
        }
        cp_async_commit();

        const uint32_t a_s = smem_u32(smem + (kt % STAGES) * STAGE_BYTES);
        const uint32_t b_s = a_s + A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t af[MI][4];
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                const int row = wm * WARP_M + mi * 16 + (lane & 15);
                ldmatrix_x4(a_s + swz(row, kk * 2 + (lane >> 4)), af[mi][0], af[mi][1], af[mi][2], af[mi][3]);
            }
#pragma unroll
            for (int np = 0; np < NI / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                const int row = wn * WARP_N + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                ldmatrix_x4(b_s + swz(row, kk * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                    mma_f16(acc[mi][2 * np], af[mi][0], af[mi][1], af[mi][2], af[mi][3], b0, b1);
                    mma_f16(acc[mi][2 * np + 1], af[mi][0], af[mi][1], af[mi][2], af[mi][3], b2, b3);
                }
            }
        }
        if (next < n_k) store_a(next, next % STAGES, fetch);
    }
    cp_async_wait<0>();

    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int o = m0 + wm * WARP_M + mi * 16 + g + half * 8;
            if (o >= n_out) continue;
            const float b = bias ? bias[o] : 0.f;
#pragma unroll
            for (int ni = 0; ni < NI; ++ni) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int t = t0 + wn * WARP_N + ni * 8 + tq * 2 + e;
                    if (t >= T) continue;
                    float v = acc[mi][ni][half * 2 + e] + b;
                    if (RESIDUAL) v += residual[(size_t)t * ldr + o];
                    Y[(size_t)t * ldy + o] = v;
                }
            }
        }
    }
}

template <int BN>
void launch_bn(const WeightView & w, const __half * x16, int ldx, int T, float * y, int ldy, const float * bias, const float * residual, int ldr,
               cudaStream_t stream) {
    constexpr int smem = STAGES * (BM * 128 + BN * 128);
    const dim3 grid((w.n_out + BM - 1) / BM, (T + BN - 1) / BN);
    if (residual) {
        static bool configured = false;
        if (!configured) {
            cudaFuncSetAttribute(gemm_q4k_mma_kernel<BN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            configured = true;
        }
        gemm_q4k_mma_kernel<BN, true><<<grid, THREADS, smem, stream>>>(w.data, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x16, ldx, T, y, ldy, bias,
                                                                      residual, ldr);
    } else {
        static bool configured = false;
        if (!configured) {
            cudaFuncSetAttribute(gemm_q4k_mma_kernel<BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            configured = true;
        }
        gemm_q4k_mma_kernel<BN, false><<<grid, THREADS, smem, stream>>>(w.data, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x16, ldx, T, y, ldy, bias,
                                                                       nullptr, 0);
    }
}

} // namespace

bool gemm_mma_supported(const WeightView & w, int ldx) {
    return w.type == GGML_Q4_K && w.n_in % 256 == 0 && ldx % 8 == 0;
}

void launch_gemm_mma(const WeightView & w, const __half * x16, int ldx, int n_tokens, float * y, int ldy, const float * bias,
                     const float * residual, int ldr, cudaStream_t stream) {
    if (n_tokens > 64) {
        launch_bn<128>(w, x16, ldx, n_tokens, y, ldy, bias, residual, ldr, stream);
    } else if (n_tokens > 16) {
        launch_bn<64>(w, x16, ldx, n_tokens, y, ldy, bias, residual, ldr, stream);
    } else {
        launch_bn<16>(w, x16, ldx, n_tokens, y, ldy, bias, residual, ldr, stream);
    }
}

} // namespace rb200
