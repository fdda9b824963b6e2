// Dequant-fused Q4_K weight GEMM on the tensor cores with f32-grade accuracy.
//
//   Y[t][o] = sum_k w[o][k] x[t][k],   w = d * (sc * q) - dmin * m        (per 32-element sub-block)
//
// Rounding weights or activations to f16 costs about 3e-4 relative error per product, which a
// 32-layer model amplifies to ~1e-1 in the logits - ten times the 1e-2 budget. This kernel
// therefore feeds the tensor cores only values that f16 holds exactly:
//   - the integer sc*q (at most 63*15 = 945) as the weight operand, formed from the nibbles with
//     one fused half2 FMA:  (1024 + q) * sc - 1024 * sc;
//   - the activation as the two-term split x = hi + lo (both f16), one MMA each;
//   - the minimum term sum_sub m_sub * (sum of x over the sub-block) as ONE extra m16n8k16 MMA
//     per 256-element super-block: A = [m_0..m_7 | m_0..m_7], B = [sx_hi ; sx_lo].
// The f16 block scales d and dmin are applied in f32 once per super-block:
//   acc += d * tmp - dmin * tmin.
// All products are exact in f32, so the result differs from an f32 dot product only by
// accumulation order. Weights stay in their GGUF block layout in HBM and are read once per CTA
// column; tiles are staged in 128B-swizzled shared memory over three cp.async stages.

#include "kernels.cuh"
#include "blocks.hpp"
#include "mma_common.cuh"

namespace rb200 {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 3;
constexpr int THREADS = 256;

// Four nibbles of a word -> four exact integers sc * q as f16, in element order.
__device__ __forceinline__ void nibbles_times_scale(uint32_t word, int hi, __half2 sc2, __half2 off2, uint32_t & out01, uint32_t & out23) {
    const uint32_t v = hi ? (word >> 4) : word;
    uint32_t a = (v & 0x000F000Fu) | 0x64006400u;          // elements 0 and 2 as 1024 + q
    uint32_t b = ((v >> 8) & 0x000F000Fu) | 0x64006400u;   // elements 1 and 3
    const __half2 ha = __hfma2(*reinterpret_cast<__half2 *>(&a), sc2, off2);
    const __half2 hb = __hfma2(*reinterpret_cast<__half2 *>(&b), sc2, off2);
    const uint32_t ua = *reinterpret_cast<const uint32_t *>(&ha), ub = *reinterpret_cast<const uint32_t *>(&hb);
    out01 = __byte_perm(ua, ub, 0x5410);
    out23 = __byte_perm(ua, ub, 0x7632);
}

struct Fetch {
    uint4 hdr, q0, q1;
};

template <int BN, bool RESIDUAL>
__global__ void __launch_bounds__(THREADS) gemm_q4k_exact_kernel(const uint8_t * __restrict__ W, int n_in, int n_out, int row_bytes, SplitAct X,
                                                                 int T, float * __restrict__ Y, int ldy, const float * __restrict__ bias,
                                                                 const float * __restrict__ residual, int ldr) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int A_BYTES = BM * 128;
    constexpr int B_BYTES = BN * 128;
    constexpr int STAGE_BYTES = A_BYTES + 2 * B_BYTES;
    constexpr int HDR_OFF = STAGES * STAGE_BYTES;          // float2 dd[2][BM]; then half m[2][BM][8]
    constexpr int WN = BN >= 64 ? 2 : 1;
    constexpr int WM = 8 / WN;
    constexpr int WARP_M = BM / WM;
    constexpr int WARP_N = BN / WN;
    constexpr int MI = WARP_M / 16;
    constexpr int NI = WARP_N / 8;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % WM, wn = warp / WM;
    const int g = lane >> 2, tq = lane & 3;
    const int m0 = blockIdx.x * BM, t0 = blockIdx.y * BN;
    const int n_k = n_in / BK;
    const int n_sub = n_in / 32;

    float2 * dd_s = reinterpret_cast<float2 *>(smem + HDR_OFF);
    __half * m_s = reinterpret_cast<__half *>(smem + HDR_OFF + 2 * BM * sizeof(float2));

    const int a_row = tid >> 1, a_half = tid & 1;
    const bool a_valid = m0 + a_row < n_out;
    const uint8_t * a_base = W + (size_t)(m0 + (a_valid ? a_row : 0)) * row_bytes;

    auto fetch_a = [&](int kt, Fetch & f) {
        if (!a_valid) return;
        const int k0 = kt * BK;
        const uint8_t * blk = a_base + (size_t)(k0 >> 8) * 144;
        f.hdr = *reinterpret_cast<const uint4 *>(blk);
        const uint4 * qs = reinterpret_cast<const uint4 *>(blk + 16 + ((k0 & 255) >> 6) * 32);
        f.q0 = qs[0];
        f.q1 = qs[1];
    };
    auto store_a = [&](int kt, int stage, const Fetch & f) {
        uint8_t * a_s = smem + stage * STAGE_BYTES;
        uint4 out[4];
        const int grp = kt & 3;                      // 64-element group inside the super-block
        if (a_valid) {
            uint32_t sc, mn;
            q4k_scale_min_regs(f.hdr, grp * 2 + a_half, sc, mn);
            const __half2 sc2 = __half2half2(__ushort2half_rn((unsigned short)sc));
            const __half2 off2 = __half2half2(__float2half_rn(-1024.0f * (float)sc));
            nibbles_times_scale(f.q0.x, a_half, sc2, off2, out[0].x, out[0].y);
            nibbles_times_scale(f.q0.y, a_half, sc2, off2, out[0].z, out[0].w);
            nibbles_times_scale(f.q0.z, a_half, sc2, off2, out[1].x, out[1].y);
            nibbles_times_scale(f.q0.w, a_half, sc2, off2, out[1].z, out[1].w);
            nibbles_times_scale(f.q1.x, a_half, sc2, off2, out[2].x, out[2].y);
            nibbles_times_scale(f.q1.y, a_half, sc2, off2, out[2].z, out[2].w);
            nibbles_times_scale(f.q1.z, a_half, sc2, off2, out[3].x, out[3].y);
            nibbles_times_scale(f.q1.w, a_half, sc2, off2, out[3].z, out[3].w);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4 *>(a_s + swz(a_row, a_half * 4 + c)) = out[c];
        if (grp == 0 && a_half == 0) {
            // first stage of a super-block: publish its d, dmin and the eight 6-bit mins
            const int slot = (kt >> 2) & 1;
            float2 dd = make_float2(0.f, 0.f);
            uint4 mv = make_uint4(0, 0, 0, 0);
            if (a_valid) {
                const __half2 h = *reinterpret_cast<const __half2 *>(&f.hdr.x);
                dd = make_float2(__low2float(h), __high2float(h));
                uint32_t mw[4];
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    uint32_t s0, n0, s1, n1;
                    q4k_scale_min_regs(f.hdr, 2 * p, s0, n0);
                    q4k_scale_min_regs(f.hdr, 2 * p + 1, s1, n1);
                    const __half2 pr = __halves2half2(__ushort2half_rn((unsigned short)n0), __ushort2half_rn((unsigned short)n1));
                    mw[p] = *reinterpret_cast<const uint32_t *>(&pr);
                }
                mv = make_uint4(mw[0], mw[1], mw[2], mw[3]);
            }
            dd_s[slot * BM + a_row] = dd;
            *reinterpret_cast<uint4 *>(m_s + (size_t)(slot * BM + a_row) * 8) = mv;
        }
    };
    auto load_b = [&](int kt, int stage) {
        const uint32_t bh_s = smem_u32(smem + stage * STAGE_BYTES + A_BYTES);
        const uint32_t bl_s = bh_s + B_BYTES;
        const int k0 = kt * BK;
#pragma unroll
        for (int i = 0; i < (BN * 8 + THREADS - 1) / THREADS; ++i) {
            const int idx = tid + i * THREADS;
            if (BN * 8 < THREADS && idx >= BN * 8) break;
            const int r = idx >> 3, c = idx & 7;
            const int t = t0 + r;
            const size_t off = (size_t)(t < T ? t : 0) * X.ld + k0 + c * 8;
            cp_async16(bh_s + swz(r, c), X.hi + off, t < T ? 16 : 0);
            cp_async16(bl_s + swz(r, c), X.lo + off, t < T ? 16 : 0);
        }
    };

    float acc[MI][NI][4], tmp[MI][NI][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < NI; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) { acc[mi][ni][e] = 0.f; tmp[mi][ni][e] = 0.f; }

    Fetch fetch;
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
        const uint32_t bh_s = a_s + A_BYTES, bl_s = bh_s + B_BYTES;
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
                const int row = wn * WARP_N + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const uint32_t boff = swz(row, kk * 2 + ((lane >> 3) & 1));
                uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
                ldmatrix_x4(bh_s + boff, h0, h1, h2, h3);
                ldmatrix_x4(bl_s + boff, l0, l1, l2, l3);
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                    mma_f16(tmp[mi][2 * np], af[mi][0], af[mi][1], af[mi][2], af[mi][3], h0, h1);
                    mma_f16(tmp[mi][2 * np + 1], af[mi][0], af[mi][1], af[mi][2], af[mi][3], h2, h3);
                    mma_f16(tmp[mi][2 * np], af[mi][0], af[mi][1], af[mi][2], af[mi][3], l0, l1);
                    mma_f16(tmp[mi][2 * np + 1], af[mi][0], af[mi][1], af[mi][2], af[mi][3], l2, l3);
                }
            }
        }
        if ((kt & 3) == 3) {
            // end of a super-block: the min term as one MMA, then the f32 block scales
            const int sb = kt >> 2, slot = sb & 1;
            uint32_t bmh[NI], bml[NI];
#pragma unroll
            for (int ni = 0; ni < NI; ++ni) {
                const int t = t0 + wn * WARP_N + ni * 8 + g;
                bmh[ni] = 0;
                bml[ni] = 0;
                if (t < T) {
                    const size_t off = (size_t)t * n_sub + sb * 8 + 2 * tq;
                    bmh[ni] = *reinterpret_cast<const uint32_t *>(X.sum_hi + off);
                    bml[ni] = *reinterpret_cast<const uint32_t *>(X.sum_lo + off);
                }
            }
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                const int r0 = wm * WARP_M + mi * 16 + g, r1 = r0 + 8;
                const float2 dd0 = dd_s[slot * BM + r0], dd1 = dd_s[slot * BM + r1];
                const uint32_t am0 = *reinterpret_cast<const uint32_t *>(m_s + (size_t)(slot * BM + r0) * 8 + 2 * tq);
                const uint32_t am1 = *reinterpret_cast<const uint32_t *>(m_s + (size_t)(slot * BM + r1) * 8 + 2 * tq);
#pragma unroll
                for (int ni = 0; ni < NI; ++ni) {
                    float tmin[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_f16(tmin, am0, am1, am0, am1, bmh[ni], bml[ni]);
                    acc[mi][ni][0] += dd0.x * tmp[mi][ni][0] - dd0.y * tmin[0];
                    acc[mi][ni][1] += dd0.x * tmp[mi][ni][1] - dd0.y * tmin[1];
                    acc[mi][ni][2] += dd1.x * tmp[mi][ni][2] - dd1.y * tmin[2];
                    acc[mi][ni][3] += dd1.x * tmp[mi][ni][3] - dd1.y * tmin[3];
                    tmp[mi][ni][0] = tmp[mi][ni][1] = tmp[mi][ni][2] = tmp[mi][ni][3] = 0.f;
                }
            }
        }
        if (next < n_k) store_a(next, next % STAGES, fetch);
    }
    cp_async_wait<0>();

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

template <int BN, bool RESIDUAL>
void launch_one(const WeightView & w, const SplitAct & x, int T, float * y, int ldy, const float * bias, const float * residual, int ldr,
                cudaStream_t stream) {
    constexpr int smem = STAGES * (BM * 128 + 2 * BN * 128) + 2 * BM * (int)sizeof(float2) + 2 * BM * 8 * (int)sizeof(__half);
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(gemm_q4k_exact_kernel<BN, RESIDUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    const dim3 grid((w.n_out + BM - 1) / BM, (T + BN - 1) / BN);
    gemm_q4k_exact_kernel<BN, RESIDUAL><<<grid, THREADS, smem, stream>>>(w.data, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x, T, y, ldy, bias,
                                                                        residual, ldr);
}

template <int BN>
void launch_bn(const WeightView & w, const SplitAct & x, int T, float * y, int ldy, const float * bias, const float * residual, int ldr,
               cudaStream_t stream) {
    if (residual) launch_one<BN, true>(w, x, T, y, ldy, bias, residual, ldr, stream);
    else launch_one<BN, false>(w, x, T, y, ldy, bias, nullptr, 0, stream);
}

} // namespace

bool gemm_q4k_exact_supported(const WeightView & w, const SplitAct & x) {
    return w.type == GGML_Q4_K && w.n_in % 256 == 0 && x.hi && x.ld == (int)w.n_in;
}

void launch_gemm_q4k_exact(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                           const float * residual, int ldr, cudaStream_t stream) {
    if (n_tokens > 64) launch_bn<128>(w, x, n_tokens, y, ldy, bias, residual, ldr, stream);
    else if (n_tokens > 16) launch_bn<64>(w, x, n_tokens, y, ldy, bias, residual, ldr, stream);
    else launch_bn<16>(w, x, n_tokens, y, ldy, bias, residual, ldr, stream);
}

} // namespace rb200
