// Dequant-fused Q8_0 weight GEMM on the 5th-generation tensor cores (tcgen05, accumulator in tensor memory),
// for steps of more than 16 tokens.
//
// Q8_0 (crates/rir-core/src/quant.rs, block of 34 bytes): an f16 scale d and 32 int8 values q; a weight is
// d * q. The product of an 11-bit and an 8-bit significand has at most 19 bits, so a weight is EXACTLY the sum of
// two f16 numbers: w_hi = round_f16(d * q) (one half2 multiply) and w_lo = d * q - w_hi (one fused half2
// multiply-add, whose single rounding has nothing to round: the remainder is a multiple of 2^-24 of at most eight
// bits). Holds for every d that keeps |d * q| inside the f16 range, checked once per matrix on the host
// (q8_0_products_fit_f16: |d| < 256 and finite); other matrices take the mma.sync kernel. With the activations as
// their two-term split x = x_hi + x_lo, a product is three MMAs
//     w_hi x_hi + w_hi x_lo + w_lo x_hi        (w_lo x_lo is below 2^-22 of the product, like the split's own rest)
// into ONE f32 accumulator that runs over the whole row: no per-block scale is left for an epilogue, so nothing
// is read back from tensor memory until the row is done.
//
// One CTA: 128 weight rows x BN tokens (128, or 256 when the grid still fills the GPU). Warps: two or three producer
// groups of four warps that take pipeline stages in turn - a warp reads the two blocks (68 bytes) of each of its 32
// rows for the stage's 64 columns straight from the GGUF row layout (coalesced along the rows, then a row per
// lane through shared memory), thread p decodes row p and stores w_hi and w_lo into lane p of the stage's two A
// slots in TENSOR MEMORY; one thread of the group fetches the activation tiles (hi and lo)
// with TMA -, eight epilogue warps, and one warp that walks the pipeline with warp-uniform values and issues
// the MMAs from an elected lane. A tile with fewer tokens than columns issues narrower MMAs (N in steps of 16).
// Tensor memory: the accumulator (BN columns), then 64 columns per stage (w_hi | w_lo, 128 rows x 64 f16 each).
// Every mbarrier wait is bounded; a wait that gives up raises the error flag and the CTA frees its tensor memory.

#include <cmath>
#include <cstdlib>
#include <cstring>

#include "kernels.cuh"
#include "blocks.hpp"
#include "mma_common.cuh"
#include "tc5_common.cuh"

namespace rb200 {

namespace {

constexpr int BM = 128;
constexpr int TMEM_COLS = 512;

// A producer warp reads the 32 x 68 bytes of its rows' stage segments as 544 consecutive-per-row words - lane after
// lane along a row, so a load instruction touches two or three rows instead of 32 - and hands every lane its own
// row's 17 words through this much shared memory (a row per lane straight from global memory costs one memory
// wavefront per lane and instruction: measured 2400 cycles per stage, against 850 of tensor work).
constexpr int kRowExchangeBytes = 32 * 17 * 4;

template <int BN> struct Shape {
    // producer groups of four warps: with 128-token tiles the producers set the pace and a third group helps
    // (0.96 against 1.05 ms on 28 672 x 4096 x 1792); with 256-token tiles the MMAs do, and a third group only
    // takes issue slots from the issuing warp (0.74 against 0.69 ms)
    static constexpr int GROUPS = BN == 256 ? 2 : 3;
    static constexpr int EPI_WARP0 = 4 * GROUPS, MMA_WARP = EPI_WARP0 + 8;
    static constexpr int THREADS = (MMA_WARP + 1) * 32;
    static constexpr int STAGES = BN == 256 ? 3 : 5;
    static constexpr int B_BYTES = BN * 128;                 // BN tokens x 64 f16, 128-byte swizzled rows
    static constexpr int STAGE_BYTES = 2 * B_BYTES;          // activation tiles hi and lo
    static constexpr int TMEM_A = BN;                        // the accumulator at column 0, then the A slots
    static constexpr int BAR_BYTES = 256;
    static constexpr int ROWS_OFF = STAGES * STAGE_BYTES + BAR_BYTES;          // the producer warps' row exchange areas
    static constexpr int SMEM_BYTES = ROWS_OFF + 4 * GROUPS * kRowExchangeBytes + 1024 /* alignment slack */;
    static_assert(TMEM_A + STAGES * 64 <= TMEM_COLS, "tensor memory: accumulator and A slots");
};

// Four int8 of a word (already XORed with 0x80: bytes u = q + 128) -> (q0, q1), (q2, q3) as f16 pairs: 0x6400 | u
// is the f16 number 1024 + u, and subtracting 1152 is exact.
__device__ __forceinline__ void int8x4_to_half2(uint32_t u, __half2 & a, __half2 & b) {
    uint32_t ua = __byte_perm(u, 0x64646464u, 0x4140), ub = __byte_perm(u, 0x64646464u, 0x4342);
    const __half2 off = __float2half2_rn(1152.0f);
    a = __hsub2(*reinterpret_cast<__half2 *>(&ua), off);
    b = __hsub2(*reinterpret_cast<__half2 *>(&ub), off);
}

template <int BN, bool RESIDUAL>
__global__ void __launch_bounds__(Shape<BN>::THREADS, 1) gemm_q8_0_tc5_kernel(const uint8_t * __restrict__ W, int n_in, int n_out, int row_bytes,
                                                                   const __grid_constant__ SplitAct X, int T, float * __restrict__ Y, int ldy,
                                                                   const float * __restrict__ bias, const float * __restrict__ residual, int ldr,
                                                                   int * __restrict__ error_flag) {
    using S = Shape<BN>;
    constexpr int STAGES = S::STAGES, B_BYTES = S::B_BYTES, STAGE_BYTES = S::STAGE_BYTES;
    constexpr int GROUPS = S::GROUPS, EPI_WARP0 = S::EPI_WARP0, MMA_WARP = S::MMA_WARP;
    extern __shared__ uint8_t smem_raw[];
    uint8_t * smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    // barriers: full[STAGES], empty[STAGES], accumulator full; then the TMEM base word and the abort flag
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);
    uint32_t * tmem_word = reinterpret_cast<uint32_t *>(smem + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 1));
    volatile int * abort_flag = reinterpret_cast<volatile int *>(tmem_word + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.y * BM, t0 = blockIdx.x * BN;   // token tiles vary fastest: CTAs in flight share a weight tile in L2
    const int n_it = n_in / 64;
    // a tile with fewer tokens than columns only pays for the columns it has, in whole MMA widths of 16
    const int mma_n = min(BN, (T - t0 + 15) & ~15);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc5::mbar_init(full_bar(s), 4);     // the producer group's warps; the TMA bytes are tracked as transactions
            tc5::mbar_init(empty_bar(s), 1);
        }
        tc5::mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        tc5::fence_mbar_init();
    }
    if (warp == MMA_WARP) tc5::tmem_alloc(smem_u32(tmem_word), TMEM_COLS);
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = *tmem_word;

    if (warp < EPI_WARP0) {
        // ------------------------------------------------------------------ producers
        const int group = warp >> 2;
        const int p = tid & 127;                       // weight row of this thread
        // The stage's two blocks of a row are 68 consecutive bytes on a 4-byte boundary: words 0..8 hold the first
        // block (scale in the low half of word 0), the high half of word 8 the second block's scale, words 9..16 its
        // values. They are prefetched two own stages ahead, so the HBM latency never holds a pipeline slot.
        struct Raw { uint32_t w[17]; };
        // word i of the warp's 544 (i = 32 k + lane) is word i % 17 of row i / 17
        const uint8_t * warp_rows = W + (size_t)(m0 + (warp & 3) * 32) * row_bytes;
        const int rows_left = n_out - (m0 + (warp & 3) * 32);
        uint32_t * exchange = reinterpret_cast<uint32_t *>(smem + S::ROWS_OFF + warp * kRowExchangeBytes);
        auto prefetch = [&](int it, Raw & raw) {
            if (it >= n_it) return;
#pragma unroll
            for (int k = 0; k < 17; ++k) {
                const int i = k * 32 + lane, r = (i * 61681) >> 20, j = i - r * 17;      // r = i / 17 for i < 544
                raw.w[k] = r < rows_left ? *reinterpret_cast<const uint32_t *>(warp_rows + (size_t)r * row_bytes + (size_t)it * 68 + j * 4) : 0u;
            }
        };
        // the lane's own row out of the warp's words
        auto own_row = [&](Raw & raw) {
#pragma unroll
            for (int k = 0; k < 17; ++k) exchange[k * 32 + lane] = raw.w[k];
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 17; ++k) raw.w[k] = exchange[lane * 17 + k];
            __syncwarp();
        };
        auto decode_store = [&](const uint32_t (&q)[8], uint32_t d_bits, uint32_t slot_hi) {
            const uint32_t dd = d_bits | (d_bits << 16);
            const __half2 d2 = *reinterpret_cast<const __half2 *>(&dd);
            uint32_t hi[16], lo[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __half2 a, b;
                int8x4_to_half2(q[i] ^ 0x80808080u, a, b);
                const __half2 ha = __hmul2(a, d2), hb = __hmul2(b, d2);
                const __half2 la = __hfma2(a, d2, __hneg2(ha)), lb = __hfma2(b, d2, __hneg2(hb));
                hi[2 * i] = *reinterpret_cast<const uint32_t *>(&ha);
                hi[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&hb);
                lo[2 * i] = *reinterpret_cast<const uint32_t *>(&la);
                lo[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&lb);
            }
            tc5::tmem_st16_nowait(slot_hi, hi);
            tc5::tmem_st16_nowait(slot_hi + 32, lo);
        };
        // returns false when the pipeline was aborted
        auto produce = [&](int it, Raw & raw) -> bool {
            const int stage = it % STAGES, use = it / STAGES;
            // warp-uniform outcome: the tensor-memory stores below are warp-collective
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(empty_bar(stage), (use & 1) ^ 1, abort_flag))) return false;
            tc5::fence_after_sync();
            if (p == 0) {
                // the activation tiles (hi and lo, BN tokens x 64 columns each, in boxes of 128 tokens) arrive by TMA
                const uint32_t bh = smem_base + stage * STAGE_BYTES, bl = bh + B_BYTES;
                tc5::mbar_expect_tx(full_bar(stage), 2 * B_BYTES);
#pragma unroll
                for (int box = 0; box < BN / 128; ++box) {
                    tc5::tma_load_2d(bh + box * 16384, &X.map_hi, it * 64, t0 + box * 128, full_bar(stage));
                    tc5::tma_load_2d(bl + box * 16384, &X.map_lo, it * 64, t0 + box * 128, full_bar(stage));
                }
            }
            const uint32_t a_slot = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + S::TMEM_A + stage * 64;
            own_row(raw);
            uint32_t q[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = __byte_perm(raw.w[i], raw.w[i + 1], 0x5432);
            decode_store(q, raw.w[0] & 0xFFFFu, a_slot);
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = raw.w[9 + i];
            decode_store(q, raw.w[8] >> 16, a_slot + 16);
            prefetch(it + 2 * GROUPS, raw);
            tc5::tmem_wait_st();                // the stage's four stores, before the barrier says they are there
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(full_bar(stage));
            return true;
        };
        Raw raw0, raw1;
        // programmatic stream serialization: only weights are touched before the wait
        prefetch(group, raw0);
        prefetch(group + GROUPS, raw1);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int it = group; it < n_it; it += 2 * GROUPS) {
            if (!produce(it, raw0)) break;
            if (it + GROUPS < n_it && !produce(it + GROUPS, raw1)) break;
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t idesc = tc5::instr_desc_f16(BM, mma_n);
        const uint64_t desc0 = tc5::smem_desc_sw128(smem_base);
        const uint32_t desc_lo0 = (uint32_t)desc0, desc_hi = (uint32_t)(desc0 >> 32);
        const uint32_t d_acc = tmem_base, a_slot0 = tmem_base + S::TMEM_A;
        int stage = 0, full_parity = 0;
        for (int it = 0; it < n_it; ++it) {
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(full_bar(stage), full_parity, abort_flag))) break;
            tc5::fence_after_sync();
            const uint32_t bh = desc_lo0 + stage * (STAGE_BYTES >> 4), bl = bh + (B_BYTES >> 4);
            const uint32_t a_hi = a_slot0 + stage * 64, a_lo = a_hi + 32;
            const uint32_t issue = tc5::elect_one() ? 1u : 0u;
            if (it == 0) {
                tc5::mma_f16_ts_pred<0>(issue, d_acc, a_hi, bh, desc_hi, idesc);
            } else {
                tc5::mma_f16_ts_pred<1>(issue, d_acc, a_hi, bh, desc_hi, idesc);
            }
            tc5::mma_f16_ts_pred<1>(issue, d_acc, a_hi, bl, desc_hi, idesc);
            tc5::mma_f16_ts_pred<1>(issue, d_acc, a_lo, bh, desc_hi, idesc);
#pragma unroll
            for (int k = 1; k < 4; ++k) {
                tc5::mma_f16_ts_pred<1>(issue, d_acc, a_hi + k * 8, bh + k * 2, desc_hi, idesc);
                tc5::mma_f16_ts_pred<1>(issue, d_acc, a_hi + k * 8, bl + k * 2, desc_hi, idesc);
                tc5::mma_f16_ts_pred<1>(issue, d_acc, a_lo + k * 8, bh + k * 2, desc_hi, idesc);
            }
            tc5::commit_pred(issue, empty_bar(stage));
            if (it == n_it - 1) tc5::commit_pred(issue, tfull_bar);
            __syncwarp();
            if (++stage == STAGES) { stage = 0; full_parity ^= 1; }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        const int colhalf = (warp - EPI_WARP0) >> 2;    // which half of the token columns
        const int o = m0 + q * 32 + lane;
        const float b = bias && o < n_out ? bias[o] : 0.f;
        if (__all_sync(0xffffffffu, tc5::mbar_wait(tfull_bar, 0, abort_flag))) {
            tc5::fence_after_sync();
            const int col0 = colhalf * (BN / 2);
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + col0;
#pragma unroll 1
            for (int c = 0; c < BN / 2; c += 32) {
                if (t0 + col0 + c >= T) break;          // warp-uniform: the rest of the tile lies past the step's tokens
                float v[16], w[16];
                tc5::tmem_ld16x2(t_acc + c, t_acc + c + 16, v, w);
                if (o < n_out) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int ta = t0 + col0 + c + i, tb = ta + 16;
                        if (ta < T) {
                            float r = v[i] + b;
                            if (RESIDUAL) r += residual[(size_t)ta * ldr + o];
                            Y[(size_t)ta * ldy + o] = r;
                        }
                        if (tb < T) {
                            float r = w[i] + b;
                            if (RESIDUAL) r += residual[(size_t)tb * ldr + o];
                            Y[(size_t)tb * ldy + o] = r;
                        }
                    }
                }
            }
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (tid == 0 && *abort_flag) atomicExch(error_flag, 1);
}

template <int BN, bool RESIDUAL>
void launch_one(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias, const float * residual, int ldr,
                int * error_flag, cudaStream_t stream) {
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) cudaFuncSetAttribute(gemm_q8_0_tc5_kernel<BN, RESIDUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<BN>::SMEM_BYTES);
    // the kernel may start (barriers, tensor-memory allocation, first weight loads) while the stream's
    // earlier kernels drain; every role waits on the device before it touches activations or outputs
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((n_tokens + BN - 1) / BN, (w.n_out + BM - 1) / BM);
    cfg.blockDim = dim3(Shape<BN>::THREADS);
    cfg.dynamicSmemBytes = Shape<BN>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, gemm_q8_0_tc5_kernel<BN, RESIDUAL>, w.data, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x, n_tokens, y, ldy, bias, residual,
                       ldr, error_flag);
}

} // namespace

bool q8_0_products_fit_f16(const uint8_t * blocks, size_t n_blocks) {
    bool ok = true;
#pragma omp parallel for reduction(&& : ok)
    for (long long b = 0; b < (long long)n_blocks; ++b) {
        uint16_t hd;
        std::memcpy(&hd, blocks + (size_t)b * 34, 2);
        const float d = half_to_float(hd);
        if (!(std::fabs(d) < 256.f)) ok = false;        // also refuses NaN and infinity
    }
    return ok;
}

bool gemm_q8_0_tc5_supported(const WeightView & w, const SplitAct & x) {
    return w.type == GGML_Q8_0 && w.tc5_exact && w.n_in % 64 == 0 && w.row_bytes % 4 == 0 && (uintptr_t)w.data % 4 == 0 && x.hi &&
           x.ld == (int)w.n_in && x.has_maps;
}

void launch_gemm_q8_0_tc5(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias, const float * residual,
                          int ldr, int * error_flag, int n_sm, cudaStream_t stream) {
    if (n_tokens <= 0) return;
    // 256-token tiles halve the decode work per product, but the grid is whole waves of one CTA per SM: the form
    // with the shorter estimated time wins (measured per 64-column stage: about 1800 cycles at N = 256, where the
    // twelve MMAs take 1536, and 1300 at N = 128, where the producers set the pace)
    const int row_tiles = (int)((w.n_out + BM - 1) / BM);
    const long long waves_wide = ((long long)row_tiles * ((n_tokens + 255) / 256) + n_sm - 1) / n_sm;
    const long long waves_narrow = ((long long)row_tiles * ((n_tokens + 127) / 128) + n_sm - 1) / n_sm;
    bool wide = n_tokens > 128 && waves_wide * 1800 < waves_narrow * 1300;
    static const int forced = [] {          // RB200_Q8_TC5_TILE=128|256 pins the form (measurements)
        const char * env = std::getenv("RB200_Q8_TC5_TILE");
        return env ? std::atoi(env) : 0;
    }();
    if (forced == 128) wide = false;
    if (forced == 256 && n_tokens > 128) wide = true;
    if (wide) {
        if (residual) launch_one<256, true>(w, x, n_tokens, y, ldy, bias, residual, ldr, error_flag, stream);
        else launch_one<256, false>(w, x, n_tokens, y, ldy, bias, nullptr, 0, error_flag, stream);
    } else {
        if (residual) launch_one<128, true>(w, x, n_tokens, y, ldy, bias, residual, ldr, error_flag, stream);
        else launch_one<128, false>(w, x, n_tokens, y, ldy, bias, nullptr, 0, error_flag, stream);
    }
}

} // namespace rb200
