// Grouped MXFP4 expert GEMM on the 5th-generation tensor cores (tcgen05, accumulator in tensor memory): the
// (token, expert) pairs of a mixture-of-experts layer, sorted by expert, times each expert's bank, one launch.
//
// MXFP4 (crates/rir-core/src/quant.rs:286-295, quant_table.rs:420-440): 32 weights in 17 bytes, an E8M0 exponent
// byte x and sixteen bytes of E2M1 nibbles (byte i holds weight i in its low and weight 16 + i in its high
// nibble); a weight is m * 2^(x - 127) with m in +-{0, .5, 1, 1.5, 2, 3, 4, 6}. Such a weight IS an f16 whenever
// 104 <= x <= 128, so the tensor cores get the weights themselves as their A operand - no block scale is left
// for an epilogue, the accumulator runs over the whole row, and the arithmetic is the exact-product scheme of the
// Q4_K kernel (activations as hi + lo, two MMAs per product, f32 accumulation) without its per-block stage.
// The decode is bit placement: the three magnitude bits of a nibble, put at bits 11..9 of an f16, are the
// number m * 2^-14 (subnormals included); the sign goes to bit 15; one half2 multiply by 2^(x - 113) finishes it.
//
// The banks are regrouped once at load (mxfp4_retile_kernel) into tiles of 128 rows x 64 columns: the rows' 32
// nibble bytes (4096 bytes, row p at 32 p), then their two exponent bytes (256 bytes): 4352 bytes per tile, the
// 17 / 32 bytes per weight of the format, and a warp that takes a row per lane reads consecutive bytes.
//
// One CTA: 128 weight rows of one expert x 128 of its pairs. Warp roles as in the Q4_K kernel: three producer
// groups of four warps (thread p decodes the 64 weights of row p into lane p of the stage's A slot in tensor
// memory; one thread fetches the activation tiles with TMA), eight epilogue warps, one issuing warp that walks
// the pipeline with warp-uniform values and an elected-lane predicate. The grid's x dimension numbers the
// (expert, token tile) items; a CTA finds its own in the offsets array. An element's arithmetic does not depend on the tile or the column it lands in,
// so results do not depend on how the pairs are grouped (nor on the expert-parallel world size).
// Every mbarrier wait is bounded; a wait that gives up raises the error flag and the CTA frees its tensor memory.

#include "kernels.cuh"
#include "blocks.hpp"
#include "mma_common.cuh"
#include "tc5_common.cuh"

namespace rb200 {

namespace {

constexpr int BM = 128;
constexpr int GROUPS = 3;
constexpr int EPI_WARP0 = 4 * GROUPS, MMA_WARP = EPI_WARP0 + 8;
constexpr int THREADS = (MMA_WARP + 1) * 32;
constexpr int TMEM_COLS = 512;
constexpr int kMaxGroups = 1024;                  // experts per launch

// Token tiles are 128 pairs wide (five pipeline stages) or 256 wide (three stages of 64 KB): with a few hundred pairs
// per expert the wide form decodes an expert's weight tile once instead of twice.
template <int BN> struct Shape {
    static constexpr int STAGES = BN == 256 ? 3 : 5;
    static constexpr int B_BYTES = BN * 128;
    static constexpr int STAGE_BYTES = 2 * B_BYTES;          // activation tiles hi and lo
    static constexpr int TMEM_A = BN;                        // the accumulator at column 0, then the A slots of 32 columns
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(TMEM_A + STAGES * 32 <= TMEM_COLS, "tensor memory: accumulator and A slots");
};

// grid (column groups of 64, row tiles, experts), 128 threads: thread p moves the two blocks of row p
__global__ void mxfp4_retile_kernel(const uint8_t * __restrict__ bank, uint32_t n_out, uint32_t n_in, uint8_t * __restrict__ tiled) {
    const uint32_t g = blockIdx.x, tile = blockIdx.y, e = blockIdx.z, p = threadIdx.x;
    const uint32_t n_groups = n_in / 64, row_tiles = gridDim.y;
    const uint32_t row = tile * 128 + p;
    uint8_t * dst = tiled + (((size_t)e * row_tiles + tile) * n_groups + g) * kMxfp4TileBytes;
    uint8_t bytes[34];
    if (row < n_out) {
        const uint8_t * src = bank + (((size_t)e * n_out + row) * (n_in / 32) + 2 * g) * 17;
#pragma unroll
        for (int i = 0; i < 34; ++i) bytes[i] = src[i];
    } else {
#pragma unroll
        for (int i = 0; i < 34; ++i) bytes[i] = 0;
        bytes[0] = bytes[17] = 113;     // scale 1: the nibbles are zero anyway
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        dst[p * 32 + i] = bytes[1 + i];
        dst[p * 32 + 16 + i] = bytes[18 + i];
    }
    dst[4096 + 2 * p] = bytes[0];
    dst[4096 + 2 * p + 1] = bytes[17];
}

// 2^(x - 113) as f16 bits, both lanes: the factor that turns the placed nibble bits into the weight.
__device__ __forceinline__ __half2 block_scale(uint32_t x) {
    const uint32_t bits = x >= 99u ? (x - 98u) << 10 : 1u << (x - 89u);
    const uint32_t both = bits | (bits << 16);
    return *reinterpret_cast<const __half2 *>(&both);
}

// Four nibbles of `t` (one per byte, already isolated in bits 3..0) -> the high bytes of four f16 values:
// magnitude bits to 3..1, sign to bit 7.
__device__ __forceinline__ uint32_t nibble_high_bytes(uint32_t t) { return ((t << 1) | (t << 4)) & 0x8E8E8E8Eu; }

// 16 nibble bytes of one block -> its 32 weights as 16 half2 in element order: out[0..7] the low nibbles
// (elements 0..15), out[8..15] the high nibbles (elements 16..31).
__device__ __forceinline__ void decode_block(const uint4 & q, __half2 scale, uint32_t * out) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t lo = nibble_high_bytes(w[j] & 0x0F0F0F0Fu);
        const uint32_t hi = ((w[j] >> 3) & 0x0E0E0E0Eu) | (w[j] & 0x80808080u);
        uint32_t a = __byte_perm(lo, 0u, 0x1404), b = __byte_perm(lo, 0u, 0x3424);       // (e0, e1), (e2, e3) as f16 pairs
        uint32_t c = __byte_perm(hi, 0u, 0x1404), d = __byte_perm(hi, 0u, 0x3424);
        const __half2 ha = __hmul2(*reinterpret_cast<__half2 *>(&a), scale), hb = __hmul2(*reinterpret_cast<__half2 *>(&b), scale);
        const __half2 hc = __hmul2(*reinterpret_cast<__half2 *>(&c), scale), hd = __hmul2(*reinterpret_cast<__half2 *>(&d), scale);
        out[2 * j] = *reinterpret_cast<const uint32_t *>(&ha);
        out[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&hb);
        out[8 + 2 * j] = *reinterpret_cast<const uint32_t *>(&hc);
        out[8 + 2 * j + 1] = *reinterpret_cast<const uint32_t *>(&hd);
    }
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1) gemm_mxfp4_tc5_kernel(const uint8_t * __restrict__ W, int n_in, int n_out, int n_groups,
                                                                    const int32_t * __restrict__ offsets, const __grid_constant__ SplitAct X,
                                                                    float * __restrict__ Y, int ldy, int * __restrict__ error_flag) {
    // blockIdx.x numbers the (expert, token tile) items expert by expert; the grid holds an upper bound of them
    // (every expert may end in a partial tile), so only the few CTAs past the last item leave empty-handed. A
    // grid of (most pairs of any expert) x experts would be mostly CTAs that find nothing to do, each of which
    // still has to wait for a whole SM's shared memory before it can say so.
    __shared__ int32_t sh_off[kMaxGroups + 1];
    for (int i = threadIdx.x; i <= n_groups; i += THREADS) sh_off[i] = offsets[i];
    __syncthreads();
    int expert = -1, t0 = 0;
    {
        int item = blockIdx.x;
        for (int e = 0; e < n_groups; ++e) {
            const int tiles = (sh_off[e + 1] - sh_off[e] + BN - 1) / BN;
            if (item < tiles) {
                expert = e;
                t0 = item * BN;
                break;
            }
            item -= tiles;
        }
    }
    if (expert < 0) return;
    const int row0 = sh_off[expert], n_rows = sh_off[expert + 1] - row0;

    using S = Shape<BN>;
    constexpr int STAGES = S::STAGES, B_BYTES = S::B_BYTES, STAGE_BYTES = S::STAGE_BYTES, TMEM_A = S::TMEM_A;
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
    const int m0 = blockIdx.y * BM;
    const int n_it = n_in / 64;
    const int row_tiles = gridDim.y;

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
        const int p = tid & 127;
        const uint8_t * tile_base = W + ((size_t)expert * row_tiles + blockIdx.y) * n_it * kMxfp4TileBytes;
        struct Raw { uint4 q0, q1; uint32_t sc; };
        auto prefetch = [&](int it, Raw & raw) {
            if (it >= n_it) return;
            const uint8_t * tile = tile_base + (size_t)it * kMxfp4TileBytes;
            const uint4 * qs = reinterpret_cast<const uint4 *>(tile + p * 32);
            raw.q0 = qs[0];
            raw.q1 = qs[1];
            raw.sc = *reinterpret_cast<const unsigned short *>(tile + 4096 + 2 * p);
        };
        auto produce = [&](int it, Raw & raw) -> bool {
            const int stage = it % STAGES, use = it / STAGES;
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(empty_bar(stage), (use & 1) ^ 1, abort_flag))) return false;
            tc5::fence_after_sync();
            if (p == 0) {
                const uint32_t bh = smem_base + stage * STAGE_BYTES, bl = bh + B_BYTES;
                tc5::mbar_expect_tx(full_bar(stage), 2 * B_BYTES);
#pragma unroll
                for (int box = 0; box < BN / 128; ++box) {      // the tensor maps' boxes are 128 rows
                    tc5::tma_load_2d(bh + box * 16384, &X.map_hi, it * 64, row0 + t0 + box * 128, full_bar(stage));
                    tc5::tma_load_2d(bl + box * 16384, &X.map_lo, it * 64, row0 + t0 + box * 128, full_bar(stage));
                }
            }
            uint32_t out[32];
            decode_block(raw.q0, block_scale(raw.sc & 0xFFu), out);
            decode_block(raw.q1, block_scale(raw.sc >> 8), out + 16);
            const uint32_t a_slot = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + TMEM_A + stage * 32;
            tc5::tmem_st32(a_slot, out);
            prefetch(it + 2 * GROUPS, raw);
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(full_bar(stage));
            return true;
        };
        Raw raw0, raw1;
        prefetch(group, raw0);
        prefetch(group + GROUPS, raw1);
        for (int it = group; it < n_it; it += 2 * GROUPS) {
            if (!produce(it, raw0)) break;
            if (it + GROUPS < n_it && !produce(it + GROUPS, raw1)) break;
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        // a tile with fewer pairs than columns (the usual case in decode steps: a few dozen pairs per expert) only
        // pays for the columns it has, in whole MMA widths of 16
        const uint32_t idesc = tc5::instr_desc_f16(BM, min(BN, (n_rows - t0 + 15) & ~15));
        const uint64_t desc0 = tc5::smem_desc_sw128(smem_base);
        const uint32_t desc_lo0 = (uint32_t)desc0, desc_hi = (uint32_t)(desc0 >> 32);
        const uint32_t d_acc = tmem_base, a_slot0 = tmem_base + TMEM_A;
        int stage = 0, full_parity = 0;
        for (int it = 0; it < n_it; ++it) {
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(full_bar(stage), full_parity, abort_flag))) break;
            tc5::fence_after_sync();
            const uint32_t bh = desc_lo0 + stage * (STAGE_BYTES >> 4), bl = bh + (B_BYTES >> 4);
            const uint32_t a_slot = a_slot0 + stage * 32;
            const uint32_t issue = tc5::elect_one() ? 1u : 0u;
            if (it == 0) {
                tc5::mma_f16_ts_pred<0>(issue, d_acc, a_slot, bh, desc_hi, idesc);
            } else {
                tc5::mma_f16_ts_pred<1>(issue, d_acc, a_slot, bh, desc_hi, idesc);
            }
            tc5::mma_f16_ts_pred<1>(issue, d_acc, a_slot, bl, desc_hi, idesc);
#pragma unroll
            for (int k = 1; k < 4; ++k) {
                tc5::mma_f16_ts_pred<1>(issue, d_acc, a_slot + k * 8, bh + k * 2, desc_hi, idesc);
                tc5::mma_f16_ts_pred<1>(issue, d_acc, a_slot + k * 8, bl + k * 2, desc_hi, idesc);
            }
            tc5::commit_pred(issue, empty_bar(stage));
            if (it == n_it - 1) tc5::commit_pred(issue, tfull_bar);
            __syncwarp();
            if (++stage == STAGES) { stage = 0; full_parity ^= 1; }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        const int colhalf = (warp - EPI_WARP0) >> 2;    // which half of the token columns
        const int o = m0 + q * 32 + lane;
        if (__all_sync(0xffffffffu, tc5::mbar_wait(tfull_bar, 0, abort_flag))) {
            tc5::fence_after_sync();
            const int col0 = colhalf * (BN / 2);
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + col0;
#pragma unroll 1
            for (int c = 0; c < BN / 2; c += 32) {
                if (t0 + col0 + c >= n_rows) break;      // warp-uniform: columns past the expert's pairs were never computed
                float v[16], w[16];
                tc5::tmem_ld16x2(t_acc + c, t_acc + c + 16, v, w);
                if (o < n_out) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int ta = t0 + col0 + c + i, tb = ta + 16;
                        if (ta < n_rows) Y[(size_t)(row0 + ta) * ldy + o] = v[i];
                        if (tb < n_rows) Y[(size_t)(row0 + tb) * ldy + o] = w[i];
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

} // namespace

bool mxfp4_scales_are_f16(const uint8_t * blocks, size_t n_blocks) {
    bool ok = true;
#pragma omp parallel for reduction(&& : ok)
    for (long long b = 0; b < (long long)n_blocks; ++b) {
        const uint8_t x = blocks[(size_t)b * 17];
        if (x < 104 || x > 128) ok = false;
    }
    return ok;
}

size_t mxfp4_tiled_bytes(uint32_t n_expert, uint32_t n_out, uint32_t n_in) {
    return (size_t)n_expert * ((n_out + 127) / 128) * (n_in / 64) * kMxfp4TileBytes;
}

void launch_mxfp4_retile(const uint8_t * bank, uint32_t n_expert, uint32_t n_out, uint32_t n_in, uint8_t * tiled, cudaStream_t stream) {
    mxfp4_retile_kernel<<<dim3(n_in / 64, (n_out + 127) / 128, n_expert), 128, 0, stream>>>(bank, n_out, n_in, tiled);
}

bool gemm_mxfp4_tc5_supported(const WeightView & w, const SplitAct & x) {
    return w.type == GGML_MXFP4 && w.tiled && w.n_in % 64 == 0 && x.hi && x.ld == (int)w.n_in && x.has_maps;
}

void launch_gemm_mxfp4_tc5_grouped(const WeightView & w, int n_groups, const int32_t * group_offsets, const SplitAct & x, int total_rows, float * y,
                                   int ldy, int * error_flag, cudaStream_t stream) {
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(gemm_mxfp4_tc5_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<128>::SMEM_BYTES);
        cudaFuncSetAttribute(gemm_mxfp4_tc5_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<256>::SMEM_BYTES);
    }
    if (n_groups <= 0 || n_groups > kMaxGroups || total_rows <= 0) return;
    // plain launches: the CTA reads its expert's offsets (written by the grouping kernel in front of it) before anything
    // else. The pairs per expert are known on the device only; their mean picks the tile width.
    if (total_rows > 96 * n_groups) {
        const dim3 grid((total_rows + 255) / 256 + n_groups, (w.n_out + BM - 1) / BM);
        gemm_mxfp4_tc5_kernel<256><<<grid, THREADS, Shape<256>::SMEM_BYTES, stream>>>(w.tiled, (int)w.n_in, (int)w.n_out, n_groups, group_offsets, x, y,
                                                                                  ldy, error_flag);
    } else {
        const dim3 grid((total_rows + 127) / 128 + n_groups, (w.n_out + BM - 1) / BM);
        gemm_mxfp4_tc5_kernel<128><<<grid, THREADS, Shape<128>::SMEM_BYTES, stream>>>(w.tiled, (int)w.n_in, (int)w.n_out, n_groups, group_offsets, x, y,
                                                                                  ldy, error_flag);
    }
}

} // namespace rb200
