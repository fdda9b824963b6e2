// Dequant-fused Q4_K weight GEMM for decode steps of at most 8 tokens: bound by the HBM stream of
// the weights, so everything is arranged around reading each weight byte once, with many bytes in
// flight per SM, and spending as few instructions per weight as possible.
//
// Arithmetic follows the exact scheme of gemm_q4k_exact.cu (integer weight operand, activations as
// hi + lo, minimum term as one extra MMA per super-block, scales, d and dmin applied in f32), on
// mma.sync m16n8k16 with the tokens as the N = 8 dimension. With at most four tokens the hi and lo
// terms of a token sit in two columns of the same MMA (columns t and t + 4), which halves the MMAs.
//
// Work split: a CTA owns a K chunk of eight 256-column super-blocks and a range of 32-row units.
// Two warps share a super-block, one per 128-column half; a warp keeps the activation fragments of
// ITS columns in registers for the whole kernel (they are the same for every weight row) and walks
// the units of the range. Each warp runs its own ring of bulk asynchronous copies (its 2560-byte half
// of a quarter tile of the tile-major weight copy per stage, completion counted on an mbarrier), so
// about 80 KB of weights are in flight per SM without holding registers. Weight nibbles go from
// shared memory into MMA A fragments: because the K order inside a fragment is free as long as both
// operands agree, and because a nibble masked in place is a valid f16 (the subnormal q * 2^-24, or
// 16 q * 2^-24 from bits 4..7), eight weights cost one shift and four logic ops, no arithmetic and
// no byte permutes; the 6-bit scale is applied in f32 to each 32-column sub-block's sum. The sixteen warps' partial sums are added
// in shared memory; partial sums per K chunk go to a small scratch array and are added in a fixed
// order (plus bias and residual) by a second tiny kernel, so results do not depend on scheduling.

#include "kernels.cuh"
#include "blocks.hpp"
#include "mma_common.cuh"
#include "tc5_common.cuh"

namespace rb200 {

namespace {

constexpr int SW = 8;                      // super-blocks per K chunk
constexpr int NWARP = 2 * SW;              // two warps per super-block
constexpr int STHREADS = NWARP * 32;
constexpr int STAGES = 3;                  // ring depth per warp
constexpr int UB = 2;                      // 32-row units per block-wide reduction
constexpr int STAGE_BYTES = 2560;          // two 64-column groups of 32 rows + their 32 headers
constexpr int RED_BYTES = 2 * UB * 2 * NWARP * 128 * 4;
constexpr int RING_BYTES = NWARP * STAGES * STAGE_BYTES;
constexpr int SMEM_BYTES = RED_BYTES + RING_BYTES + NWARP * STAGES * 8 + 16;

// Plain (untiled) bulk copy global -> shared, no multicast; completion in bytes on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

struct UnitRaw {
    uint4 hdr0, hdr1;      // block headers of rows g and g + 8
    uint2 q0[2], q1[2];    // per 64-column group of this warp's half: words 2tq, 2tq+1 of the two rows
};

// PACK4: at most four tokens; MMA column t carries the hi term of token t, column t + 4 its lo term.
template <bool PACK4>
__global__ void __launch_bounds__(STHREADS, 1) gemm_q4k_stream_kernel(const uint8_t * __restrict__ Wt, int n_in, int n_out, SplitAct X, int T,
                                                                      float * __restrict__ partial, int units_per_cta, int * __restrict__ error_flag) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    float * red = reinterpret_cast<float *>(smem_raw);                       // [2][UB * 2][NWARP][128]
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t ring_base = smem_base + RED_BYTES;
    const uint32_t bar_base = ring_base + RING_BYTES;
    volatile int * abort_flag = reinterpret_cast<volatile int *>(smem_raw + RED_BYTES + RING_BYTES + NWARP * STAGES * 8);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int n_sb = n_in / 256, n_sub = n_in / 32;
    const int kchunk = blockIdx.y;
    const int sb = kchunk * SW + (warp >> 1);
    const int kh = warp & 1;                       // which 128-column half of the super-block
    const bool sb_valid = sb < n_sb;
    const int n_units = (n_out + 31) / 32;
    const int u_begin = blockIdx.x * units_per_cta;
    const int u_end = min(n_units, u_begin + units_per_cta);
    const uint32_t my_ring = ring_base + warp * STAGES * STAGE_BYTES;
    const uint32_t my_bars = bar_base + warp * STAGES * 8;

    if (tid == 0) *abort_flag = 0;
    if (lane == 0) {
        for (int s2 = 0; s2 < STAGES; ++s2) tc5::mbar_init(my_bars + s2 * 8, 1);
        tc5::fence_mbar_init();
    }
    __syncthreads();

    // unit u: quarter (u % 4) of row tile (u / 4); half 0 = [group 0 | group 1 | headers], half 1 = [headers | group 2 | group 3]
    auto issue = [&](int u, int stage) {
        const uint8_t * src = Wt + ((size_t)(u >> 2) * n_sb + sb) * kQ4kTileBytes + (size_t)(u & 3) * kQ4kQuarterBytes + (kh ? 2048 : 0);
        tc5::mbar_arrive_expect_tx(my_bars + stage * 8, STAGE_BYTES);
        bulk_load(my_ring + stage * STAGE_BYTES, src, STAGE_BYTES, my_bars + stage * 8);
    };
    if (sb_valid && lane == 0) {
        for (int s2 = 0; s2 < STAGES; ++s2)
            if (u_begin + s2 < u_end) issue(u_begin + s2, s2);
    }
    // Launched with programmatic stream serialization: everything above touches only the weights, which
    // no kernel writes, so it may run while the kernels before this one are still finishing. From here on
    // the activations are read and results written: wait for every earlier kernel of the stream.
    // The finish kernel that follows is launched the same way and may be scheduled from now on (it
    // waits for this kernel's completion before it reads the partial sums).
    pdl_trigger();
    pdl_wait();

    // ---- this warp's activation fragments: MMA column g, K steps of its 128 columns
    uint32_t bh[8][2], bl[8][2], bmh = 0, bml = 0;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) bh[ks][0] = bh[ks][1] = bl[ks][0] = bl[ks][1] = 0;
    {
        const int tok = PACK4 ? (g & 3) : g;
        if (sb_valid && tok < T) {
            const size_t row = (size_t)tok * X.ld + (size_t)sb * 256 + (size_t)kh * 128;
            const __half * src_a = (PACK4 && g >= 4) ? X.lo : X.hi;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                // K step ks = sub-block ks / 2 of the half, word ks % 2: elements 4 (2 tq + ks % 2) .. + 3 of the sub-block
                const int e = (ks >> 1) * 32 + 4 * (2 * tq + (ks & 1));
                const uint2 vh = *reinterpret_cast<const uint2 *>(src_a + row + e);
                bh[ks][0] = __byte_perm(vh.x, vh.y, 0x5410);     // elements 0, 2
                bh[ks][1] = __byte_perm(vh.x, vh.y, 0x7632);     // elements 1, 3
                if (!PACK4) {
                    const uint2 vl = *reinterpret_cast<const uint2 *>(X.lo + row + e);
                    bl[ks][0] = __byte_perm(vl.x, vl.y, 0x5410);
                    bl[ks][1] = __byte_perm(vl.x, vl.y, 0x7632);
                }
            }
            if (!PACK4 || g < 4) {
                bmh = *reinterpret_cast<const uint32_t *>(X.sum_hi + (size_t)tok * n_sub + sb * 8 + 2 * tq);
                bml = *reinterpret_cast<const uint32_t *>(X.sum_lo + (size_t)tok * n_sub + sb * 8 + 2 * tq);
            }
        }
    }

    // rows 16 h + g and 16 h + g + 8 of the staged half quarter
    const int hdr_off = kh ? 0 : 2048, grp_off = kh ? 512 : 0;
    auto read_stage = [&](int stage, int h, UnitRaw & raw) {
        const uint8_t * base = smem_raw + RED_BYTES + (warp * STAGES + stage) * STAGE_BYTES;
        const int p0 = 16 * h + g;
        raw.hdr0 = *reinterpret_cast<const uint4 *>(base + hdr_off + p0 * 16);
        raw.hdr1 = *reinterpret_cast<const uint4 *>(base + hdr_off + (p0 + 8) * 16);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            raw.q0[j] = *reinterpret_cast<const uint2 *>(base + grp_off + j * 1024 + p0 * 32 + 8 * tq);
            raw.q1[j] = *reinterpret_cast<const uint2 *>(base + grp_off + j * 1024 + (p0 + 8) * 32 + 8 * tq);
        }
    };

    // lane constants of the minimum-term fragment: which word of the packed minimums holds bytes
    // 2 tq and 2 tq + 1, and the byte selector that turns them into two f16 values 1024 + m
    const bool min_upper = tq >= 2;
    const uint32_t min_sel = 0x4040u | (((2 * tq) & 3) + 1) << 8 | ((2 * tq) & 3);
    const __half2 k1024 = __float2half2_rn(1024.f);

    // the unit's contribution of this warp's 128 columns: rows g / g+8 x MMA columns 2tq, 2tq+1
    auto compute = [&](const UnitRaw & raw, int h, float (&part)[4]) {
        // The four 6-bit scales of this half (sub-blocks 4 kh .. 4 kh + 3), one per byte, unpacked with
        // byte-parallel logic; no integer-to-float conversion instructions anywhere.
        const uint32_t sc0 = kh ? ((raw.hdr0.w & 0x0F0F0F0Fu) | ((raw.hdr0.y >> 2) & 0x30303030u)) : (raw.hdr0.y & 0x3F3F3F3Fu);
        const uint32_t sc1 = kh ? ((raw.hdr1.w & 0x0F0F0F0Fu) | ((raw.hdr1.y >> 2) & 0x30303030u)) : (raw.hdr1.y & 0x3F3F3F3Fu);
        // A scale byte placed in the low mantissa bits of the f32 2^23 reads as 2^23 + sc; under 2^19 as 2^19 + sc / 16.
        auto scale_lo = [&](uint32_t packed, int j) -> float { return __uint_as_float(__byte_perm(packed, 0x4B000000u, 0x7540u | j)) - 8388608.f; };
        auto scale_hi = [&](uint32_t packed, int j) -> float { return __uint_as_float(__byte_perm(packed, 0x49000000u, 0x7540u | j)) - 524288.f; };
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            // group j of the half: sub-block 2j in the low nibbles, 2j + 1 in the high nibbles. The MMA's
            // weight operand is the masked nibble itself: as an f16 bit pattern q in bits 0..3 is the
            // subnormal q * 2^-24 and q in bits 4..7 is 16 q * 2^-24, both exact.
            float alo[4], ahi[4];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const uint32_t wa = hh ? raw.q0[j].y : raw.q0[j].x, wb = hh ? raw.q1[j].y : raw.q1[j].x;     // rows g, g + 8
                const uint32_t ua = wa >> 8, ub = wb >> 8;
                const uint32_t l0 = wa & 0x000F000Fu, l1 = wb & 0x000F000Fu, l2 = ua & 0x000F000Fu, l3 = ub & 0x000F000Fu;
                const uint32_t h0 = wa & 0x00F000F0u, h1 = wb & 0x00F000F0u, h2 = ua & 0x00F000F0u, h3 = ub & 0x00F000F0u;
                const int ks_lo = 4 * j + hh, ks_hi = 4 * j + 2 + hh;
                if (hh == 0) {
                    mma_f16_first(alo, l0, l1, l2, l3, bh[ks_lo][0], bh[ks_lo][1]);
                    mma_f16_first(ahi, h0, h1, h2, h3, bh[ks_hi][0], bh[ks_hi][1]);
                } else {
                    mma_f16(alo, l0, l1, l2, l3, bh[ks_lo][0], bh[ks_lo][1]);
                    mma_f16(ahi, h0, h1, h2, h3, bh[ks_hi][0], bh[ks_hi][1]);
                }
                if (!PACK4) {
                    mma_f16(alo, l0, l1, l2, l3, bl[ks_lo][0], bl[ks_lo][1]);
                    mma_f16(ahi, h0, h1, h2, h3, bl[ks_hi][0], bl[ks_hi][1]);
                }
            }
            const float sl0 = scale_lo(sc0, 2 * j), sl1 = scale_lo(sc1, 2 * j), sh0 = scale_hi(sc0, 2 * j + 1), sh1 = scale_hi(sc1, 2 * j + 1);
            // two fused multiply-adds per result (not a product, a fused multiply-add and an addition)
            tot[0] = fmaf(sh0, ahi[0], fmaf(sl0, alo[0], tot[0]));
            tot[1] = fmaf(sh0, ahi[1], fmaf(sl0, alo[1], tot[1]));
            tot[2] = fmaf(sh1, ahi[2], fmaf(sl1, alo[2], tot[2]));
            tot[3] = fmaf(sh1, ahi[3], fmaf(sl1, alo[3], tot[3]));
        }
        const __half2 dd0 = *reinterpret_cast<const __half2 *>(&raw.hdr0.x), dd1 = *reinterpret_cast<const __half2 *>(&raw.hdr1.x);
        const float d0 = __low2float(dd0) * 16777216.f, d1 = __low2float(dd1) * 16777216.f;      // undoes the 2^-24 of the nibbles
        part[0] = d0 * tot[0];
        part[1] = d0 * tot[1];
        part[2] = d1 * tot[2];
        part[3] = d1 * tot[3];
        if (kh == h) {
            // minimum term of the whole super-block: A = [m_0..m_7 | m_0..m_7], B = [sum_hi | sum_lo]. Both
            // warps of the super-block hold the headers; each takes it for one of the unit's two 16-row halves.
            const uint32_t mnA0 = raw.hdr0.z & 0x3F3F3F3Fu, mnB0 = ((raw.hdr0.w >> 4) & 0x0F0F0F0Fu) | ((raw.hdr0.z >> 2) & 0x30303030u);
            const uint32_t mnA1 = raw.hdr1.z & 0x3F3F3F3Fu, mnB1 = ((raw.hdr1.w >> 4) & 0x0F0F0F0Fu) | ((raw.hdr1.z >> 2) & 0x30303030u);
            const uint32_t v0 = __byte_perm(min_upper ? mnB0 : mnA0, 0x64646464u, min_sel);
            const uint32_t v1 = __byte_perm(min_upper ? mnB1 : mnA1, 0x64646464u, min_sel);
            const __half2 h0 = __hsub2(*reinterpret_cast<const __half2 *>(&v0), k1024), h1 = __hsub2(*reinterpret_cast<const __half2 *>(&v1), k1024);
            const uint32_t am0 = *reinterpret_cast<const uint32_t *>(&h0), am1 = *reinterpret_cast<const uint32_t *>(&h1);
            float tmin[4];
            mma_f16_first(tmin, am0, am1, am0, am1, bmh, bml);
            const float dm0 = __high2float(dd0), dm1 = __high2float(dd1);
            part[0] -= dm0 * tmin[0];
            part[1] -= dm0 * tmin[1];
            part[2] -= dm1 * tmin[2];
            part[3] -= dm1 * tmin[3];
        }
    };

    int buf = 0, it = 0;
    bool alive = true;
    for (int ub = u_begin; ub < u_end; ub += UB) {
#pragma unroll
        for (int j = 0; j < UB; ++j) {
            const int u = ub + j;
            const bool work = u < u_end && sb_valid && alive;
            const int stage = it % STAGES;
            bool ok = true;
            if (work) ok = tc5::mbar_wait(my_bars + stage * 8, (it / STAGES) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) alive = false;      // warp-uniform
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float part[4] = {0.f, 0.f, 0.f, 0.f};
                if (work && alive) {
                    UnitRaw raw;
                    read_stage(stage, h, raw);
                    compute(raw, h, part);
                }
                *reinterpret_cast<float4 *>(&red[(((buf * UB + j) * 2 + h) * NWARP + warp) * 128 + lane * 4]) = make_float4(part[0], part[1], part[2], part[3]);
            }
            if (work) {
                __syncwarp();       // every lane has read the stage before it is refilled
                if (lane == 0 && alive && u + STAGES < u_end) issue(u + STAGES, stage);
                ++it;
            }
        }
        __syncthreads();
        // add the sixteen warps' contributions in warp order and store the K chunk's partial sums:
        // one thread per (unit of the batch, 16-row half, fragment slot)
        {
            const int jh = tid >> 7, v = tid & 127;
            const int u = ub + (jh >> 1);
            const int ln = v >> 2, e = v & 3;
            const int t = 2 * (ln & 3) + (e & 1);
            if (u < u_end && t < T) {
                const float * src = &red[(buf * UB * 2 + jh) * NWARP * 128 + v];
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < NWARP; ++w) sum += src[w * 128];
                if (PACK4) {       // the lo terms sit four MMA columns to the right: lane tq + 2
                    float lo = 0.f;
#pragma unroll
                    for (int w = 0; w < NWARP; ++w) lo += src[w * 128 + 8];
                    sum += lo;
                }
                const int o = u * 32 + (jh & 1) * 16 + (ln >> 2) + ((e >> 1) << 3);
                if (o < n_out) partial[((size_t)kchunk * 8 + t) * n_out + o] = sum;
            }
        }
        buf ^= 1;       // the next batch writes the other buffer; one barrier per batch is enough
    }
    // A wait that gave up: say so, and give this warp's copies still in flight a bounded time to land
    // before the shared memory is released.
    if (!alive || *abort_flag) {
        if (lane == 0) {
            atomicExch(error_flag, 1);
            if (sb_valid) {
                const long long start = clock64();
                for (int s2 = 0; s2 < STAGES; ++s2) {
                    const int consumed = (it + STAGES - 1 - s2) / STAGES;      // completed phases of this stage so far
                    while (!tc5::mbar_try_wait(my_bars + s2 * 8, consumed & 1) && clock64() - start < (1ll << 28)) {}
                }
            }
        }
    }
}

} // namespace

bool gemm_q4k_stream_supported(const WeightView & w, const SplitAct & x, int n_tokens) {
    return w.type == GGML_Q4_K && w.tiled && w.n_in % 256 == 0 && x.hi && x.ld == (int)w.n_in && n_tokens >= 1 && n_tokens <= 8;
}

size_t gemm_q4k_stream_scratch_floats(uint32_t n_out, uint32_t n_in) {
    const size_t n_chunks = (n_in / 256 + SW - 1) / SW;
    return n_chunks * 8 * (size_t)n_out;
}

void launch_gemm_q4k_stream(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                            const float * residual, int ldr, float * scratch, int n_sm, int * error_flag, cudaStream_t stream,
                            const FinishTail * tail) {
    const int n_sb = (int)w.n_in / 256;
    const int n_chunks = (n_sb + SW - 1) / SW;
    const int n_units = ((int)w.n_out + 31) / 32;
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(gemm_q4k_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_q4k_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    }
    // one CTA per SM in total
    int ctas_x = max(1, n_sm / n_chunks);
    const int units_per_cta = (n_units + ctas_x - 1) / ctas_x;
    ctas_x = (n_units + units_per_cta - 1) / units_per_cta;
    const dim3 grid(ctas_x, n_chunks);
    // the kernel may start while the stream's earlier kernels drain (it waits on the device before it reads activations)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(STHREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (n_tokens <= 4) cudaLaunchKernelEx(&cfg, gemm_q4k_stream_kernel<true>, w.tiled, (int)w.n_in, (int)w.n_out, x, n_tokens, scratch, units_per_cta, error_flag);
    else cudaLaunchKernelEx(&cfg, gemm_q4k_stream_kernel<false>, w.tiled, (int)w.n_in, (int)w.n_out, x, n_tokens, scratch, units_per_cta, error_flag);
    launch_gemm_stream_finish(scratch, n_chunks, (int)w.n_out, n_tokens, 8, y, ldy, bias, residual, ldr, stream, tail);
}

} // namespace rb200
