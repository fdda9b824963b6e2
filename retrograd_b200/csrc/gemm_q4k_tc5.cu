// Dequant-fused Q4_K weight GEMM on the 5th-generation tensor cores (tcgen05, accumulators in
// tensor memory). Per 256-element super-block of a weight row
//   acc += d * ( sum_k (sc*q)_k * (x_hi + x_lo)_k  -  sum_sub (rho * m_sub) * sum_x_sub ),   rho = dmin / d.
// The tensor cores only ever see values f16 holds exactly: the integers sc*q <= 945, the two-term
// activation splits, and the minimum term's factor rho * m_sub as an f16 pair (hi + lo, 22 bits; rho is
// one f32 division per row and super-block, so the minimum term carries a relative error of ~3e-7
// instead of none - far below the f32 rounding of the sum it joins). d is applied in f32 by the
// epilogue warps. Folding the minimum term into the main accumulator this way (instead of giving it an
// accumulator of its own, scaled by dmin) frees a quarter of the tensor memory for pipeline slots. A
// matrix qualifies when every super-block has d != 0 or dmin * m == 0, and |rho * m| stays far inside
// the f16 range (q4k_min_fold_ok, checked once at load); other matrices take the mma.sync kernel.
//
// One CTA computes 128 weight rows x 128 tokens. Warp roles (21 warps):
//   0-11       three producer groups of four warps, taking pipeline stages in turn (the decode is a
//              dependent instruction chain per thread: with two groups the producers were busy 92 % of
//              the time and the issuing warp waited for them a third of it); thread p decodes the 64 weights of
//              row p and stores them into lane p of the stage's A slot in TENSOR MEMORY (the MMA reads
//              its A operand from there, so shared memory carries the activations only); one thread
//              of the group fetches the two activation tiles (hi and lo) with TMA, whose bytes
//              complete on the stage's barrier;
//   20         walks the pipeline as a whole warp (uniform address arithmetic); one elected lane issues
//              the MMAs (M 128, N 128, K 16) and commits them to the stage's "empty" barrier, and per
//              super-block to the accumulator's "full" barrier;
//   12-19      epilogue: each thread owns one weight row and 64 token columns, pulls the TMEM
//              accumulator of a finished super-block with tcgen05.ld and folds it, times d, into its
//              f32 running sums while the tensor cores already work on the next super-block in the
//              other buffer.
// Tensor memory (512 columns): two accumulators (2 x 128) and the pipeline's A slots of 32 columns
// (128 rows x 64 f16). The pipeline is five stages deep (shared memory: 5 x 32 KB of activation
// tiles); measured on 28 672 x 4096 x 2048 with three producer groups: three stages 0.88 ms, four
// 0.77, five 0.75-0.76, six 0.79, seven 0.81.
// A super-block is five pipeline stages: four of 64 columns each (eight MMAs: hi and lo), then one
// that carries the minimum term as two K=16 steps (A = [-rho*m hi | -rho*m lo], B = [sum_hi | sum_hi],
// then the same A with B = [sum_lo | sum_lo]).
// The warp that issues the MMAs is one dependent instruction stream sharing its scheduler with four
// busy warps, so its loop is kept to an add per operand and the MMA itself (descriptors are built
// once), and every other wait sleeps in hardware (try_wait with a time hint) instead of spinning.
// Barrier arrivals are one per warp (after a warp-level synchronisation), not one per thread.
// Every mbarrier wait is bounded: after about a second without progress the CTA raises an error
// flag, drains its copies, frees its tensor memory and returns.

#include <algorithm>

#include "kernels.cuh"
#include "blocks.hpp"
#include "mma_common.cuh"
#include "tc5_common.cuh"

namespace rb200 {

namespace {

constexpr int BM = 128, BN = 128;
#ifndef RB200_TC5_STAGES
#define RB200_TC5_STAGES 5
#endif
constexpr int STAGES = RB200_TC5_STAGES;
constexpr int B_BYTES = BN * 128;
constexpr int STAGE_BYTES = 2 * B_BYTES;          // activation tiles hi and lo; the weight tile lives in tensor memory
#ifndef RB200_TC5_GROUPS
#define RB200_TC5_GROUPS 3
#endif
constexpr int GROUPS = RB200_TC5_GROUPS;          // producer groups of four warps
constexpr int EPI_WARP0 = 4 * GROUPS, MMA_WARP = EPI_WARP0 + 8;
constexpr int N_WARPS = MMA_WARP + 1;
constexpr int THREADS = N_WARPS * 32;
constexpr int TMEM_COLS = 512;
constexpr int TMEM_A = 256;                    // column offsets: accumulators at 0 and 128, then the A slots
static_assert(STAGES >= 2 && STAGES <= 8, "the A slots share 256 tensor-memory columns");
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

__device__ __forceinline__ void nibbles_times_scale(uint32_t word, int hi, __half2 sc2, __half2 off2, uint32_t & out01, uint32_t & out23) {
    const uint32_t v = hi ? (word >> 4) : word;
    uint32_t a = (v & 0x000F000Fu) | 0x64006400u;
    uint32_t b = ((v >> 8) & 0x000F000Fu) | 0x64006400u;
    const __half2 ha = __hfma2(*reinterpret_cast<__half2 *>(&a), sc2, off2);
    const __half2 hb = __hfma2(*reinterpret_cast<__half2 *>(&b), sc2, off2);
    const uint32_t ua = *reinterpret_cast<const uint32_t *>(&ha), ub = *reinterpret_cast<const uint32_t *>(&hb);
    out01 = __byte_perm(ua, ub, 0x5410);
    out23 = __byte_perm(ua, ub, 0x7632);
}

// grid (super-blocks, row tiles), 128 threads: thread p moves the 144-byte block of row p
__global__ void q4k_retile_kernel(const uint8_t * __restrict__ rows, uint32_t n_out, uint32_t n_sb, uint32_t row_bytes, uint8_t * __restrict__ tiled) {
    const uint32_t sb = blockIdx.x, tile = blockIdx.y, p = threadIdx.x;
    const uint32_t row = tile * 128 + p;
    uint8_t * dst = tiled + ((size_t)tile * n_sb + sb) * kQ4kTileBytes;
    uint4 v[9];
    if (row < n_out) {
        const uint4 * src = reinterpret_cast<const uint4 *>(rows + (size_t)row * row_bytes + (size_t)sb * 144);
#pragma unroll
        for (int i = 0; i < 9; ++i) v[i] = src[i];
    } else {
#pragma unroll
        for (int i = 0; i < 9; ++i) v[i] = make_uint4(0, 0, 0, 0);
    }
    *reinterpret_cast<uint4 *>(dst + q4k_tile_hdr_offset(p)) = v[0];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        uint4 * q = reinterpret_cast<uint4 *>(dst + q4k_tile_group_offset(p, r));
        q[0] = v[1 + 2 * r];
        q[1] = v[2 + 2 * r];
    }
}

// SPLIT: the split-K form (blockIdx.z ranges over the reduction, results go to `partial`); a separate
// instantiation, so that the plain form keeps exactly the code it had before the split form existed
// (sharing one body cost the plain form 10 % in the engine).
template <bool RESIDUAL, bool SPLIT>
__global__ void __launch_bounds__(THREADS, 1) gemm_q4k_tc5_kernel(const uint8_t * __restrict__ W, int n_in, int n_out, int row_bytes,
                                                                  const __grid_constant__ SplitAct X, int T, float * __restrict__ Y, int ldy, const float * __restrict__ bias,
                                                                  const float * __restrict__ residual, int ldr, int * __restrict__ error_flag,
                                                                  int sb_per_split, float * __restrict__ partial) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t * smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    // barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then the TMEM base word and the abort flag
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    uint32_t * tmem_word = reinterpret_cast<uint32_t *>(smem + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));
    volatile int * abort_flag = reinterpret_cast<volatile int *>(tmem_word + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.y * BM, t0 = blockIdx.x * BN;   // token tiles vary fastest: CTAs in flight share a weight tile in L2
    // split-K: blockIdx.z owns super-blocks [sb0, sb0 + n_sb) of the row and writes a partial result
    const int n_sb_all = n_in / 256;
    const int sb0 = SPLIT ? blockIdx.z * sb_per_split : 0;
    const int n_sb = SPLIT ? min(n_sb_all, sb0 + sb_per_split) - sb0 : n_sb_all;
    const int n_it = n_sb * 5;
    const int n_sub = n_in / 32;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc5::mbar_init(full_bar(s), 4);     // the producer group's warps; the TMA bytes are tracked as transactions
            tc5::mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc5::mbar_init(tfull_bar(b), 1);
            tc5::mbar_init(tempty_bar(b), 8);   // the epilogue warps
        }
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
        const int p = tid & 127;                       // weight row and token row of this thread
        // (the tiled layout is zero-padded to whole row tiles: every row p exists)
        const uint8_t * tile_base = W + ((size_t)blockIdx.y * n_sb_all + sb0) * kQ4kTileBytes;
        const int t = t0 + p;
        const bool t_valid = t < T;
        // Raw block bytes are prefetched into registers two own stages ahead, so the HBM latency of
        // the weights never holds a pipeline slot; a slot is only held for the L2 latency of the
        // activation copy, which overlaps the decode.
        struct Raw { uint4 hdr, q0, q1; };
        auto prefetch = [&](int it, Raw & raw) {
            if (it >= n_it) return;
            const int sb = it / 5, r = it % 5;
            const uint8_t * blk = tile_base + (size_t)sb * kQ4kTileBytes;
            raw.hdr = *reinterpret_cast<const uint4 *>(blk + q4k_tile_hdr_offset(p));      // consecutive threads, consecutive bytes
            if (r < 4) {
                const uint4 * qs = reinterpret_cast<const uint4 *>(blk + q4k_tile_group_offset(p, r));
                raw.q0 = qs[0];
                raw.q1 = qs[1];
            } else {
                raw.q0 = raw.q1 = make_uint4(0, 0, 0, 0);
                if (t_valid) {
                    raw.q0 = *reinterpret_cast<const uint4 *>(X.sum_hi + (size_t)t * n_sub + (sb0 + sb) * 8);
                    raw.q1 = *reinterpret_cast<const uint4 *>(X.sum_lo + (size_t)t * n_sub + (sb0 + sb) * 8);
                }
            }
        };
        // returns false when the pipeline was aborted
        auto produce = [&](int it, Raw & raw) -> bool {
            const int stage = it % STAGES, use = it / STAGES;
            // warp-uniform outcome: the tensor-memory stores below are warp-collective
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(empty_bar(stage), (use & 1) ^ 1, abort_flag))) return false;
            tc5::fence_after_sync();
            const int sb = it / 5, r = it % 5;
            uint8_t * bh_s = smem + stage * STAGE_BYTES;
            const uint32_t a_slot = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + TMEM_A + stage * 32;
            if (r < 4) {
                if (p == 0) {
                    // the activation tiles (hi and lo, 128 tokens x 64 columns each) arrive by TMA
                    const uint32_t bh = smem_u32(bh_s), bl = bh + B_BYTES;
                    tc5::mbar_expect_tx(full_bar(stage), 2 * B_BYTES);
                    tc5::tma_load_2d(bh, &X.map_hi, (sb0 + sb) * 256 + r * 64, t0, full_bar(stage));
                    tc5::tma_load_2d(bl, &X.map_lo, (sb0 + sb) * 256 + r * 64, t0, full_bar(stage));
                }
                // 64 weights -> 32 columns of f16 pairs in K order: low nibbles (columns 0..31 of the group), then high
                uint32_t out[32];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t sc, mn;
                    q4k_scale_min_regs(raw.hdr, r * 2 + half, sc, mn);
                    const __half2 sc2 = __half2half2(__ushort2half_rn((unsigned short)sc));
                    const __half2 off2 = __half2half2(__float2half_rn(-1024.0f * (float)sc));
                    uint32_t * o = out + half * 16;
                    nibbles_times_scale(raw.q0.x, half, sc2, off2, o[0], o[1]);
                    nibbles_times_scale(raw.q0.y, half, sc2, off2, o[2], o[3]);
                    nibbles_times_scale(raw.q0.z, half, sc2, off2, o[4], o[5]);
                    nibbles_times_scale(raw.q0.w, half, sc2, off2, o[6], o[7]);
                    nibbles_times_scale(raw.q1.x, half, sc2, off2, o[8], o[9]);
                    nibbles_times_scale(raw.q1.y, half, sc2, off2, o[10], o[11]);
                    nibbles_times_scale(raw.q1.z, half, sc2, off2, o[12], o[13]);
                    nibbles_times_scale(raw.q1.w, half, sc2, off2, o[14], o[15]);
                }
                tc5::tmem_st32(a_slot, out);
                prefetch(it + 2 * GROUPS, raw);
            } else {
                // minimum-term stage: A = [-rho*m_0..7 hi | lo], B tiles [sum_hi | sum_hi] and [sum_lo | sum_lo]
                const __half2 dd = *reinterpret_cast<const __half2 *>(&raw.hdr.x);
                const float d = __low2float(dd), dmin = __high2float(dd);
                const float nrho = d != 0.f ? -dmin / d : 0.f;
                uint32_t mw[8];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t s0, n0, s1, n1;
                    q4k_scale_min_regs(raw.hdr, 2 * q, s0, n0);
                    q4k_scale_min_regs(raw.hdr, 2 * q + 1, s1, n1);
                    const float v0 = nrho * (float)n0, v1 = nrho * (float)n1;
                    const __half h0 = __float2half_rn(v0), h1 = __float2half_rn(v1);
                    const __half2 hi2 = __halves2half2(h0, h1);
                    const __half2 lo2 = __halves2half2(__float2half_rn(v0 - __half2float(h0)), __float2half_rn(v1 - __half2float(h1)));
                    mw[q] = *reinterpret_cast<const uint32_t *>(&hi2);
                    mw[q + 4] = *reinterpret_cast<const uint32_t *>(&lo2);
                }
                tc5::tmem_st8(a_slot, mw);
                *reinterpret_cast<uint4 *>(bh_s + swz(p, 0)) = raw.q0;
                *reinterpret_cast<uint4 *>(bh_s + swz(p, 1)) = raw.q0;
                *reinterpret_cast<uint4 *>(bh_s + B_BYTES + swz(p, 0)) = raw.q1;
                *reinterpret_cast<uint4 *>(bh_s + B_BYTES + swz(p, 1)) = raw.q1;
                tc5::fence_proxy_async();
                prefetch(it + 2 * GROUPS, raw);
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(full_bar(stage));
            return true;
        };
        Raw raw0, raw1;
        // Programmatic stream serialization: only weights may be touched before the wait. A minimum-term
        // stage prefetches the token's sub-block sums - activations, written by the kernel in front of this
        // one - so such a stage among the first two waits its turn.
        static_assert(GROUPS < 4, "the first stage of every group must be a weight stage");
        const bool sums_first = (group + GROUPS) % 5 == 4;
        prefetch(group, raw0);
        if (!sums_first) prefetch(group + GROUPS, raw1);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (sums_first) prefetch(group + GROUPS, raw1);
        for (int it = group; it < n_it; it += 2 * GROUPS) {
            if (!produce(it, raw0)) break;
            if (it + GROUPS < n_it && !produce(it + GROUPS, raw1)) break;
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        asm volatile("griddepcontrol.wait;" ::: "memory");
        {
            // The whole warp walks this loop with warp-uniform values; the election's outcome rides on each MMA
            // and commit as a predicate, so nothing here branches on it and the descriptor arithmetic stays
            // uniform. (With a single thread inside a divergent branch the issuing thread - not the tensor
            // pipe - set the pace: 0.94 -> 0.81 ms on 28 672 x 4096 x 2048.) Descriptors are built once; a
            // stage costs an add per operand and the MMAs themselves.
            // the step's last token tile only pays for the columns it has, in whole MMA widths of 16
            const uint32_t idesc = tc5::instr_desc_f16(BM, min(BN, (T - t0 + 15) & ~15));
            const uint64_t desc0 = tc5::smem_desc_sw128(smem_base);
            const uint32_t desc_lo0 = (uint32_t)desc0, desc_hi = (uint32_t)(desc0 >> 32);
            const uint32_t a_slot0 = tmem_base + TMEM_A;
            int stage = 0, full_parity = 0;
            bool alive = true;
            for (int sb = 0; sb < n_sb && alive; ++sb) {
                const int buf = sb & 1;
                const uint32_t d_main = tmem_base + buf * 128;
                if (!__all_sync(0xffffffffu, tc5::mbar_wait(tempty_bar(buf), ((sb >> 1) & 1) ^ 1, abort_flag))) break;
                tc5::fence_after_sync();
#pragma unroll
                for (int r = 0; r < 5; ++r) {
                    if (!__all_sync(0xffffffffu, tc5::mbar_wait(full_bar(stage), full_parity, abort_flag))) { alive = false; break; }
                    tc5::fence_after_sync();
                    const uint32_t bh = desc_lo0 + stage * (STAGE_BYTES >> 4), bl = bh + (B_BYTES >> 4);
                    const uint32_t a_slot = a_slot0 + stage * 32;
                    const uint32_t issue = tc5::elect_one() ? 1u : 0u;
                    if (r < 4) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (r == 0 && k == 0) tc5::mma_f16_ts_pred<0>(issue, d_main, a_slot, bh, desc_hi, idesc);
                            else tc5::mma_f16_ts_pred<1>(issue, d_main, a_slot + k * 8, bh + k * 2, desc_hi, idesc);
                            tc5::mma_f16_ts_pred<1>(issue, d_main, a_slot + k * 8, bl + k * 2, desc_hi, idesc);
                        }
                        tc5::commit_pred(issue, empty_bar(stage));
                    } else {
                        tc5::mma_f16_ts_pred<1>(issue, d_main, a_slot, bh, desc_hi, idesc);
                        tc5::mma_f16_ts_pred<1>(issue, d_main, a_slot, bl, desc_hi, idesc);
                        tc5::commit_pred(issue, empty_bar(stage));
                        tc5::commit_pred(issue, tfull_bar(buf));
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; full_parity ^= 1; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        const int colhalf = (warp - EPI_WARP0) >> 2;    // which 64 token columns
        const int o_local = q * 32 + lane;
        const int o = m0 + o_local;
        const bool o_valid = o < n_out;
        const uint8_t * hdr_base = W + ((size_t)blockIdx.y * n_sb_all + sb0) * kQ4kTileBytes + q4k_tile_hdr_offset(o_local);
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.f;
        bool alive = true;
        // d of the next super-block is fetched while the tensor cores still work on it
        __half2 h_next = *reinterpret_cast<const __half2 *>(hdr_base);      // (rows are padded to whole tiles)
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16) + colhalf * 64;
        for (int sb = 0; sb < n_sb && alive; ++sb) {
            const int buf = sb & 1, buse = sb >> 1;
            const float d = __low2float(h_next);
            if (sb + 1 < n_sb) h_next = *reinterpret_cast<const __half2 *>(hdr_base + (size_t)(sb + 1) * kQ4kTileBytes);
            // warp-uniform outcome: the tensor-memory loads below are warp-collective
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(tfull_bar(buf), buse & 1, abort_flag))) { alive = false; break; }
            tc5::fence_after_sync();
            const uint32_t t_main = t_lane + buf * 128;
#pragma unroll
            for (int c = 0; c < 4; c += 2) {
                float v[16], w[16];
                tc5::tmem_ld16x2(t_main + c * 16, t_main + (c + 1) * 16, v, w);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    acc[c * 16 + i] += d * v[i];
                    acc[(c + 1) * 16 + i] += d * w[i];
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(tempty_bar(buf));
        }
        if (alive && o_valid) {
            const float b = bias ? bias[o] : 0.f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const int t = t0 + colhalf * 64 + i;
                if (t < T) {
                    if (SPLIT) {
                        partial[((size_t)blockIdx.z * T + t) * n_out + o] = acc[i];      // bias and residual are added by the finish kernel
                    } else {
                        float v = acc[i] + b;
                        if (RESIDUAL) v += residual[(size_t)t * ldr + o];
                        Y[(size_t)t * ldy + o] = v;
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

namespace {
typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                             const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn tensor_map_encoder() {
    static EncodeFn encode = nullptr;
    static bool looked = false;
    if (!looked) {
        looked = true;
        void * fn = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess) {
            encode = reinterpret_cast<EncodeFn>(fn);
        }
    }
    return encode;
}
} // namespace

bool tensor_maps_available() { return tensor_map_encoder() != nullptr; }

bool split_act_encode_maps(SplitAct & s, size_t rows) {
    const EncodeFn encode = tensor_map_encoder();
    s.has_maps = 0;
    if (!encode || !s.hi || s.ld % 64 != 0 || rows == 0) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)s.ld, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)s.ld * sizeof(__half)};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t elem[2] = {1, 1};
    for (int which = 0; which < 2; ++which) {
        const CUresult r = encode(which ? &s.map_lo : &s.map_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, which ? (void *)s.lo : (void *)s.hi, dims,
                                  strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return false;
    }
    s.has_maps = 1;
    return true;
}

bool attention_maps_encode(AttentionMaps & maps, const __half * k, const __half * v, int head_dim, uint64_t rows) {
    const EncodeFn encode = tensor_map_encoder();
    maps.valid = 0;
    if (!encode || !k || !v || head_dim % 64 != 0 || rows == 0 || rows > 0x7fffffffull) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)head_dim * sizeof(__half)};
    const cuuint32_t box[2] = {64, 16};
    const cuuint32_t elem[2] = {1, 1};
    for (int which = 0; which < 2; ++which) {
        const CUresult r = encode(which ? &maps.v : &maps.k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, which ? (void *)v : (void *)k, dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return false;
    }
    maps.valid = 1;
    return true;
}

bool gemm_q4k_tc5_supported(const WeightView & w, const SplitAct & x) {
    return w.type == GGML_Q4_K && w.tiled && w.tc5_exact && w.n_in % 256 == 0 && x.hi && x.ld == (int)w.n_in && x.has_maps;
}

bool q4k_min_fold_ok(const uint8_t * blocks, size_t n_blocks) {
    bool ok = true;
#pragma omp parallel for reduction(&& : ok)
    for (long long b = 0; b < (long long)n_blocks; ++b) {
        const uint8_t * blk = blocks + (size_t)b * 144;
        uint16_t hd, hm;
        std::memcpy(&hd, blk, 2);
        std::memcpy(&hm, blk + 2, 2);
        const float d = half_to_float(hd), dmin = half_to_float(hm);
        if (!std::isfinite(d) || !std::isfinite(dmin)) {
            ok = false;
            continue;
        }
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, mn;
            q4k_scale_min(j, blk + 4, sc, mn);
            if (d == 0.f ? dmin * (float)mn != 0.f : !(std::fabs(dmin / d * (float)mn) < 16384.f)) ok = false;
        }
    }
    return ok;
}

void launch_q4k_retile(const uint8_t * rows, uint32_t n_out, uint32_t n_in, uint32_t row_bytes, uint8_t * tiled, cudaStream_t stream) {
    q4k_retile_kernel<<<dim3(n_in / 256, (n_out + 127) / 128), 128, 0, stream>>>(rows, n_out, n_in / 256, row_bytes, tiled);
}

void launch_gemm_q4k_tc5(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                         const float * residual, int ldr, int * error_flag, float * scratch, size_t scratch_floats, int n_sm, cudaStream_t stream,
                         const FinishTail * tail) {
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(gemm_q4k_tc5_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_q4k_tc5_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_q4k_tc5_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    }
    // few output tiles (few tokens and few rows): cut the reduction into splits of whole super-blocks so the
    // grid still covers the GPU; the splits' partial results are added, in order, by the finish kernel
    const int n_sb = (int)w.n_in / 256;
    int splits = scratch ? gemm_q4k_tc5_splits(w.n_out, w.n_in, n_tokens, n_sm) : 1;
    if ((size_t)splits * n_tokens * w.n_out > scratch_floats) splits = 1;
    const int sb_per_split = (n_sb + splits - 1) / splits;
    float * partial = splits > 1 ? scratch : nullptr;
    const dim3 grid((n_tokens + BN - 1) / BN, (w.n_out + BM - 1) / BM, splits);
    // the kernel may start (barriers, tensor-memory allocation, first weight loads) while the stream's
    // earlier kernels drain; every role waits on the device before it touches activations or outputs
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float * no_residual = nullptr;
    if (splits > 1) {
        // bias and residual are the finish kernel's
        cudaLaunchKernelEx(&cfg, gemm_q4k_tc5_kernel<false, true>, w.tiled, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x, n_tokens, y, ldy, bias,
                           no_residual, 0, error_flag, sb_per_split, partial);
    } else if (residual) {
        cudaLaunchKernelEx(&cfg, gemm_q4k_tc5_kernel<true, false>, w.tiled, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x, n_tokens, y, ldy, bias, residual,
                           ldr, error_flag, sb_per_split, partial);
    } else {
        cudaLaunchKernelEx(&cfg, gemm_q4k_tc5_kernel<false, false>, w.tiled, (int)w.n_in, (int)w.n_out, (int)w.row_bytes, x, n_tokens, y, ldy, bias,
                           no_residual, 0, error_flag, sb_per_split, partial);
    }
    if (splits > 1) launch_gemm_stream_finish(scratch, splits, (int)w.n_out, n_tokens, n_tokens, y, ldy, bias, residual, ldr, stream, tail);
}

int gemm_q4k_tc5_splits(uint32_t n_out, uint32_t n_in, int n_tokens, int n_sm) {
    const int n_sb = (int)n_in / 256;
    const int tiles = ((n_tokens + BN - 1) / BN) * (int)((n_out + BM - 1) / BM);
    if (tiles * 2 > n_sm) return 1;
    const int want = std::min(n_sm / tiles, n_sb / 2);
    if (want <= 1) return 1;
    const int sb_per_split = (n_sb + want - 1) / want;
    return (n_sb + sb_per_split - 1) / sb_per_split;
}

size_t gemm_q4k_tc5_scratch_floats(uint32_t n_out, uint32_t n_in, int n_tokens, int n_sm) {
    const int splits = gemm_q4k_tc5_splits(n_out, n_in, n_tokens, n_sm);
    return splits > 1 ? (size_t)splits * n_tokens * n_out : 0;
}

} // namespace rb200
