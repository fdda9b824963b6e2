// Dequant-fused Q8_0 weight GEMM on the tensor cores (mma.sync.m16n8k16) with f32-grade accuracy, for
// steps of more than 8 tokens:
//
//   Y[t][o] = sum_blocks d[o][b] * sum_{k in block b} q[o][k] x[t][k]
//
// The tensor cores only see values f16 holds exactly: the int8 weight as an integer (one XOR, one byte
// permute and one half2 add per two weights), the activation as the two-term split x = hi + lo. A
// 32-column block is exactly two K steps, so its sum lands in a temporary accumulator of its own and
// the block's f16 scale d is applied in f32: acc += d * tmp. Weights stay in their GGUF block layout
// (34 bytes per 32 weights) and are decoded once per CTA into 128B-swizzled shared memory over three
// stages; the activation tiles arrive with cp.async.

#include "kernels.cuh"
#include "blocks.hpp"
#include "mma_common.cuh"

namespace rb200 {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;          // two Q8_0 blocks per stage
constexpr int STAGES = 3;
constexpr int THREADS = 256;

struct Fetch {
    uint32_t w[9];              // nine words covering the thread's 34-byte block (d, then 32 int8), which starts at
                                // halfword 0 (first block of the stage) or halfword 1 (second block) of the window
};

template <int BN, bool RESIDUAL>
__global__ void __launch_bounds__(THREADS) gemm_q8_0_exact_kernel(const uint8_t * __restrict__ W, int n_in, int n_out, int row_bytes, SplitAct X,
                                                                  int T, float * __restrict__ Y, int ldy, const float * __restrict__ bias,
                                                                  const float * __restrict__ residual, int ldr,
                                                                  const int32_t * __restrict__ group_offsets, unsigned long long group_stride) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int A_BYTES = BM * 128;
    constexpr int B_BYTES = BN * 128;
    constexpr int STAGE_BYTES = A_BYTES + 2 * B_BYTES;
    constexpr int D_OFF = STAGES * STAGE_BYTES;            // float d[STAGES][2][BM]
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
    if (group_offsets) {
        // grouped form: blockIdx.z is a group (an expert) with its own weight matrix and its own contiguous
        // range of activation / result rows; the grid's token tiles are an upper bound
        const int begin = group_offsets[blockIdx.z];
        T = group_offsets[blockIdx.z + 1] - begin;
        if (t0 >= T) return;
        W += (size_t)blockIdx.z * group_stride;
        X.hi += (size_t)begin * X.ld;
        X.lo += (size_t)begin * X.ld;
        Y += (size_t)begin * ldy;
    }

    float * d_s = reinterpret_cast<float *>(smem + D_OFF);

    const int a_row = tid >> 1, a_half = tid & 1;          // this thread decodes block a_half of the stage for row a_row
    const bool a_valid = m0 + a_row < n_out;
    const uint8_t * a_base = W + (size_t)(m0 + (a_valid ? a_row : 0)) * row_bytes;

    auto fetch_a = [&](int kt, Fetch & f) {
        if (!a_valid) return;
        // a stage's two blocks of a row are 68 consecutive bytes starting on a 4-byte boundary (rows are whole
        // pairs of blocks): the first block is words 0..8, the second the upper half of word 8 and words 9..16
        const uint32_t * seg = reinterpret_cast<const uint32_t *>(a_base + (size_t)kt * 68) + a_half * 8;
#pragma unroll
        for (int i = 0; i < 9; ++i) f.w[i] = seg[i];
    };
    auto store_a = [&](int stage, const Fetch & f) {
        uint8_t * a_s = smem + stage * STAGE_BYTES;
        uint4 out[4];
        float d = 0.f;
        if (a_valid) {
            // the block's halfwords 2m, 2m + 1 as one word, whichever half of the window it starts in
            uint32_t p[9];
#pragma unroll
            for (int m = 0; m < 8; ++m) p[m] = __funnelshift_r(f.w[m], f.w[m + 1], 16 * a_half);
            p[8] = f.w[8] >> (16 * a_half);
            const __half dh = __ushort_as_half((unsigned short)(p[0] & 0xFFFFu));
            d = __half2float(dh);
            const __half2 k1152 = __float2half2_rn(1152.f);
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                // bytes (q0, q1) -> (q0 + 128, q1 + 128) under the f16 exponent pattern 0x64 = 1024 + byte; minus 1152
                const int j = 1 + i;                                   // halfword of the block
                const uint32_t u = p[j >> 1] ^ 0x80808080u;
                const uint32_t v = __byte_perm(u, 0x64646464u, (j & 1) ? 0x4342 : 0x4140);
                const __half2 h = __hsub2(*reinterpret_cast<const __half2 *>(&v), k1152);
                o[i] = *reinterpret_cast<const uint32_t *>(&h);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) out[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4 *>(a_s + swz(a_row, a_half * 4 + c)) = out[c];
        d_s[(stage * 2 + a_half) * BM + a_row] = d;
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
            store_a(s, fetch);
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

        const int stage = kt % STAGES;
        const uint32_t a_s = smem_u32(smem + stage * STAGE_BYTES);
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
            if (kk & 1) {
                // end of a 32-column block: its f16 scale in f32, per weight row
                const int blk = kk >> 1;
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                    const int r0 = wm * WARP_M + mi * 16 + g;
                    const float d0 = d_s[(stage * 2 + blk) * BM + r0], d1 = d_s[(stage * 2 + blk) * BM + r0 + 8];
#pragma unroll
                    for (int ni = 0; ni < NI; ++ni) {
                        acc[mi][ni][0] += d0 * tmp[mi][ni][0];
                        acc[mi][ni][1] += d0 * tmp[mi][ni][1];
                        acc[mi][ni][2] += d1 * tmp[mi][ni][2];
                        acc[mi][ni][3] += d1 * tmp[mi][ni][3];
                        tmp[mi][ni][0] = tmp[mi][ni][1] = tmp[mi][ni][2] = tmp[mi][ni][3] = 0.f;
                    }
                }
            }
        }
        if (next < n_k) store_a(next % STAGES, fetch);
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
    constexpr int smem = STAGES * (BM * 128 + 2 * BN * 128) + STAGES * 2 * BM * (int)sizeof(float);
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(gemm_q8_0_exact_kernel<BN, RESIDUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    const dim3 grid((w.n_out + BM - 1) / BM, (T + BN - 1) / BN);
    gemm_q8_0_exact_kernel<BN, RESIDUAL><<<grid, THREADS, smem, stream>>>(w.data, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x, T, y, ldy, bias,
                                                                         residual, ldr, nullptr, 0ull);
}

template <int BN>
void launch_bn(const WeightView & w, const SplitAct & x, int T, float * y, int ldy, const float * bias, const float * residual, int ldr,
               cudaStream_t stream) {
    if (residual) launch_one<BN, true>(w, x, T, y, ldy, bias, residual, ldr, stream);
    else launch_one<BN, false>(w, x, T, y, ldy, bias, nullptr, 0, stream);
}

} // namespace

bool gemm_q8_0_exact_supported(const WeightView & w, const SplitAct & x) {
    // rows of whole block pairs on 4-byte boundaries: the weight loads are 32-bit
    return w.type == GGML_Q8_0 && w.n_in % 64 == 0 && x.hi && x.ld == (int)w.n_in && w.row_bytes % 4 == 0 &&
           (reinterpret_cast<uintptr_t>(w.data) & 3) == 0;
}

void launch_gemm_q8_0_exact_grouped(const WeightView & w, uint64_t group_stride_bytes, int n_groups, const int32_t * group_offsets, const SplitAct & x,
                                    int max_group_rows, float * y, int ldy, cudaStream_t stream) {
    constexpr int BN = 64;
    constexpr int smem = STAGES * (BM * 128 + 2 * BN * 128) + STAGES * 2 * BM * (int)sizeof(float);
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(gemm_q8_0_exact_kernel<BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    if (n_groups <= 0 || max_group_rows <= 0) return;
    const dim3 grid((w.n_out + BM - 1) / BM, (max_group_rows + BN - 1) / BN, n_groups);
    gemm_q8_0_exact_kernel<BN, false><<<grid, THREADS, smem, stream>>>(w.data, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x, 0, y, ldy, nullptr, nullptr,
                                                                       0, group_offsets, (unsigned long long)group_stride_bytes);
}

void launch_gemm_q8_0_exact(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                            const float * residual, int ldr, cudaStream_t stream) {
    if (n_tokens > 64) launch_bn<128>(w, x, n_tokens, y, ldy, bias, residual, ldr, stream);
    else if (n_tokens > 16) launch_bn<64>(w, x, n_tokens, y, ldy, bias, residual, ldr, stream);
    else launch_bn<16>(w, x, n_tokens, y, ldy, bias, residual, ldr, stream);
}

} // namespace rb200
