// Paged attention for prefill chunks on the 5th-generation tensor cores (tcgen05): scores and outputs are
// accumulated in tensor memory, K/V tiles are staged from the paged cache with TMA.
//
// A CTA serves one work item = (up to 128 / G consecutive tokens of one step row) x (one KV head), G = query
// heads per KV head: 128 query vectors (token, head-in-group), one per tensor-memory lane. The slot's KV blocks
// (16 tokens x head_dim f16, contiguous per KV head) are found through the block table and fetched four at a time
// - a tile of 64 keys - by `cp.async.bulk.tensor.2d` boxes of 16 rows x 64 columns with the 128-byte swizzle,
// straight into the layouts the MMAs read: K as a K-major operand (keys x dims), V as an MN-major operand of the
// same bytes (no transpose anywhere). Per tile:
//   S = Q_hi K^T + Q_lo K^T          (SS MMAs, M 128, N 64, K 16 per step; Q staged once in shared memory)
//   softmax threads (two per query vector) pull their row of S out of tensor memory, mask by position,
//   keep the running maximum and sum, and store P = exp(S - max) as the two-term split P_hi + P_lo back
//   into tensor memory as the A operand of
//   O += P_hi V + P_lo V             (TS MMAs, M 128, N head_dim, K 16 per step)
// O is rescaled in tensor memory only in a tile where some row's maximum rose (a warp-uniform decision; in a
// long context that is the first few tiles). S and P are double-buffered, so the tensor cores compute the next
// tile's scores while the softmax threads work on this one.
//
// Accuracy as in the mma.sync kernel it replaces: K and V are exact f16 operands by storage; the query
// (pre-scaled by 1/sqrt(head_dim)) and the probabilities are two-term splits, so every product is exact in f32.
// Warps: 0 fetches, 1 issues the MMAs, 2-9 are the softmax threads (tensor-memory lane quarter = warp % 4): two per
// query vector, each with half of a tile's keys and half of O's columns; they exchange the halves' maxima per tile
// (and the sums once, at the end) through shared memory and an mbarrier.
// Every mbarrier wait is bounded; a wait that gives up raises the error flag and the CTA frees its tensor memory.

#include "kernels.cuh"
#include "mma_common.cuh"
#include "tc5_common.cuh"

#include <cfloat>

namespace rb200 {

namespace {

constexpr int ROWS = kAttentionTileRows;     // 128 query vectors per CTA
constexpr int KT = 64;                       // keys per tile: four KV blocks
constexpr int STAGES = 3;
constexpr int THREADS = 10 * 32;              // warp 0 fetches, warp 1 issues, warps 2-9 are the softmax threads
constexpr int TMEM_COLS = 512;
constexpr int TMEM_S = 0, TMEM_P = 128, TMEM_O = 256;      // S: 2 x 64 columns, P: 2 x (32 hi + 32 lo), O: head_dim

template <int HD> struct Shape {
    static constexpr int PANELS = HD / 64;                   // 128-byte panels per row
    static constexpr int Q_BYTES = PANELS * ROWS * 128;      // one of Q_hi, Q_lo
    static constexpr int KV_BYTES = PANELS * KT * 128;       // one of K, V of a stage
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int BAR_OFF = 2 * Q_BYTES + STAGES * STAGE_BYTES;
    static constexpr int XCH_OFF = BAR_OFF + 256;            // the softmax halves' exchange: 6 x 128 floats
    static constexpr int SMEM_BYTES = XCH_OFF + 6 * ROWS * 4 + 1024 /* alignment slack */;
};

// MN-major operand of [K rows][64 x f16] panels with the 128-byte swizzle: `lbo` bytes between the 64-element
// panels of the MN direction, 1024 bytes between groups of eight K rows.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 1) attention_tc5_kernel(const float * __restrict__ qkv, int ld, int n_head, KvLayout kv, int layer,
                                                                   const __grid_constant__ AttentionMaps maps, const int2 * __restrict__ items,
                                                                   const int32_t * __restrict__ tok_slot, const int32_t * __restrict__ tok_pos,
                                                                   const int32_t * __restrict__ tok_pos_min, float * __restrict__ out, int ldo,
                                                                   int skip_small, int * __restrict__ error_flag) {
    using S = Shape<HD>;
    constexpr int PANELS = S::PANELS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hk = blockIdx.y;
    const int G = n_head / kv.n_head_kv;
    // items are listed in row order (decode rows first, long prefill chunks last): walk them backwards so the
    // longest-running CTAs start first
    const int2 item = items[gridDim.x - 1 - blockIdx.x];
    const int i0 = item.x, ntok = item.y;
    if (skip_small && ntok * G <= 16) return;       // served by the split-KV kernel

    extern __shared__ uint8_t smem_raw[];
    uint8_t * smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    uint8_t * q_hi = smem;
    uint8_t * q_lo = smem + S::Q_BYTES;
    const uint32_t kv_base = smem_base + 2 * S::Q_BYTES;
    const uint32_t bar_base = smem_base + S::BAR_OFF;
    auto kv_full = [&](int s) { return bar_base + 8u * s; };
    auto kv_empty = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto s_full = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto s_free = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    auto p_full = [&](int b) { return bar_base + 8u * (2 * STAGES + 4 + b); };
    auto pv_done = [&](int b) { return bar_base + 8u * (2 * STAGES + 6 + b); };
    auto x_full = [&](int b) { return bar_base + 8u * (2 * STAGES + 8 + b); };
    const uint32_t l_full = bar_base + 8u * (2 * STAGES + 10);
    uint32_t * tmem_word = reinterpret_cast<uint32_t *>(smem + S::BAR_OFF + 8 * (2 * STAGES + 11));
    volatile int * abort_flag = reinterpret_cast<volatile int *>(tmem_word + 1);

    const int slot = tok_slot[i0], pos0 = tok_pos[i0], pmin = tok_pos_min[i0];
    const int last = pos0 + ntok - 1;
    const int nb0 = pmin >> 4, nb1 = last >> 4;
    const int n_blocks = nb1 - nb0 + 1;
    const int n_tiles = (n_blocks + 3) >> 2;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc5::mbar_init(kv_full(s), 1);
            tc5::mbar_init(kv_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc5::mbar_init(s_full(b), 1);
            tc5::mbar_init(s_free(b), 8);       // the softmax warps
            tc5::mbar_init(p_full(b), 8);
            tc5::mbar_init(pv_done(b), 1);
            tc5::mbar_init(x_full(b), 8);
        }
        tc5::mbar_init(l_full, 8);
        *abort_flag = 0;
        tc5::fence_mbar_init();
    }
    if (warp == 1) tc5::tmem_alloc(smem_u32(tmem_word), TMEM_COLS);

    // ---- stage the query tile as hi + lo f16 (every thread: 128 rows x two halves)
    {
        const float scale = rsqrtf((float)HD);
        for (int u = tid; u < 2 * ROWS; u += THREADS) {
            const int R = u >> 1, part = u & 1;
            const int tt = R / G, hg = R % G;
            const bool valid = tt < ntok;
            const float * src = qkv + (size_t)(i0 + (valid ? tt : 0)) * ld + (size_t)(hk * G + hg) * HD + part * (HD / 2);
#pragma unroll
            for (int c = 0; c < HD / 16; ++c) {          // chunks of 8 columns in this half row
                float v[8];
                if (valid) {
                    const float4 a = *reinterpret_cast<const float4 *>(src + c * 8);
                    const float4 b = *reinterpret_cast<const float4 *>(src + c * 8 + 4);
                    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = 0.f;
                }
                uint32_t h[4], l[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x0 = v[2 * e] * scale, x1 = v[2 * e + 1] * scale;
                    const __half2 hh = __floats2half2_rn(x0, x1);
                    const float2 back = __half22float2(hh);
                    h[e] = *reinterpret_cast<const uint32_t *>(&hh);
                    l[e] = pack_half2(x0 - back.x, x1 - back.y);
                }
                const int col_chunk = part * (HD / 16) + c;         // 16-byte chunk index in the row
                const uint32_t off = (uint32_t)((col_chunk >> 3) * (ROWS * 128)) + swz(R, col_chunk & 7);
                *reinterpret_cast<uint4 *>(q_hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4 *>(q_lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
            }
        }
    }
    tc5::fence_proxy_async();            // the MMAs read the query tiles through the async proxy
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = *tmem_word;

    if (warp == 0) {
        // ------------------------------------------------------------------ K/V tiles by TMA
        if (lane == 0) {
            const int32_t * table = kv.block_table + (size_t)slot * kv.max_blocks;
            const int rows_per_layer = (int)(kv.layer_stride / HD);
            for (int j = 0; j < n_tiles; ++j) {
                const int stage = j % STAGES, use = j / STAGES;
                if (!tc5::mbar_wait(kv_empty(stage), (use & 1) ^ 1, abort_flag)) break;
                const uint32_t k_s = kv_base + stage * S::STAGE_BYTES, v_s = k_s + S::KV_BYTES;
                tc5::mbar_arrive_expect_tx(kv_full(stage), 2 * S::KV_BYTES);
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    // past the sequence's last block the previous block is fetched again: its keys are masked by
                    // position, and its values are finite
                    const int bi = min(4 * j + b, n_blocks - 1);
                    const int blk = rb_block(kv, table[nb0 + bi]);
                    const int y = layer * rows_per_layer + (blk * kv.n_head_kv + hk) * 16;
#pragma unroll
                    for (int p = 0; p < PANELS; ++p) {
                        tc5::tma_load_2d(k_s + p * (KT * 128) + b * 2048, &maps.k, p * 64, y, kv_full(stage));
                        tc5::tma_load_2d(v_s + p * (KT * 128) + b * 2048, &maps.v, p * 64, y, kv_full(stage));
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc_s = tc5::instr_desc_f16(ROWS, KT);
            const uint32_t idesc_o = tc5::instr_desc_f16(ROWS, HD) | (1u << 16);       // B operand MN-major
            const uint32_t d_o = tmem_base + TMEM_O;
            bool alive = true;
            auto issue_pv = [&](int j) -> bool {
                const int b = j & 1, stage = j % STAGES;
                if (!tc5::mbar_wait(p_full(b), (j >> 1) & 1, abort_flag)) return false;
                tc5::fence_after_sync();
                const uint32_t v_s = kv_base + stage * S::STAGE_BYTES + S::KV_BYTES;
                const uint32_t p_hi = tmem_base + TMEM_P + b * 64, p_lo = p_hi + 32;
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    const uint64_t vd = smem_desc_sw128_mn(v_s + kk * 2048, KT * 128);
                    tc5::mma_f16_ts(d_o, p_hi + kk * 8, vd, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                    tc5::mma_f16_ts(d_o, p_lo + kk * 8, vd, idesc_o, 1u);
                }
                tc5::commit(kv_empty(stage));       // the stage's K and V have been read
                tc5::commit(pv_done(b));            // P buffer b is free, O holds this tile
                return true;
            };
            for (int j = 0; j < n_tiles && alive; ++j) {
                const int b = j & 1, stage = j % STAGES;
                if (!tc5::mbar_wait(kv_full(stage), (j / STAGES) & 1, abort_flag)) { alive = false; break; }
                if (!tc5::mbar_wait(s_free(b), ((j >> 1) & 1) ^ 1, abort_flag)) { alive = false; break; }
                tc5::fence_after_sync();
                const uint32_t k_s = kv_base + stage * S::STAGE_BYTES;
                const uint32_t d_s = tmem_base + TMEM_S + b * 64;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t q_off = (uint32_t)((ks >> 2) * (ROWS * 128) + (ks & 3) * 32);
                    const uint64_t kd = tc5::smem_desc_sw128(k_s + (ks >> 2) * (KT * 128) + (ks & 3) * 32);
                    tc5::mma_f16_ss(d_s, tc5::smem_desc_sw128(smem_base + q_off), kd, idesc_s, ks > 0 ? 1u : 0u);
                    tc5::mma_f16_ss(d_s, tc5::smem_desc_sw128(smem_base + S::Q_BYTES + q_off), kd, idesc_s, 1u);
                }
                tc5::commit(s_full(b));
                // the previous tile's P V, once its probabilities are in tensor memory
                if (j > 0 && !issue_pv(j - 1)) { alive = false; break; }
            }
            if (alive && n_tiles > 0) issue_pv(n_tiles - 1);
        }
    } else {
        // ------------------------------------------------------------------ softmax: two threads per query vector,
        // each with half of a tile's keys (warps 2-5 the first 32, warps 6-9 the last 32) and half of O's columns
        const int grp = (warp - 2) >> 2;
        const int q = warp & 3;
        const int R = q * 32 + lane;
        const int tt = R / G, hg = R % G;
        const int prow = tt < ntok ? pos0 + tt : -1;        // last position this query vector may see
        const int warp_min_prow = __reduce_min_sync(0xffffffffu, prow);      // (-1 with a row past the item's tokens in the warp)
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        float * xmax = reinterpret_cast<float *>(smem + S::XCH_OFF);     // [tile parity][group][row]: the halves' maxima
        float * xsum = xmax + 4 * ROWS;                                  // [group][row]: the halves' sums, at the end
        constexpr int KH = KT / 2, OH = HD / 2;
        float m = -INFINITY, l = 0.f;
        bool alive = true;
        for (int j = 0; j < n_tiles && alive; ++j) {
            const int b = j & 1;
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(s_full(b), (j >> 1) & 1, abort_flag))) { alive = false; break; }
            tc5::fence_after_sync();
            float s[KH];
            {
                float v[16], w[16];
                tc5::tmem_ld16x2(t_lane + TMEM_S + b * 64 + grp * KH, t_lane + TMEM_S + b * 64 + grp * KH + 16, v, w);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    s[i] = v[i];
                    s[16 + i] = w[i];
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(s_free(b));
            // causal mask by position within the slot; a tile whose keys every row of the warp sees (all but the first
            // and the last few tiles of a chunk) skips the per-key comparisons
            const int pbase = (nb0 << 4) + j * KT + grp * KH;
            float mx = -INFINITY;
            if (pbase >= pmin && pbase + KH - 1 <= warp_min_prow) {
#pragma unroll
                for (int i = 0; i < KH; ++i) mx = fmaxf(mx, s[i]);
            } else {
#pragma unroll
                for (int i = 0; i < KH; ++i) {
                    const int p = pbase + i;
                    if (p < pmin || p > prow) s[i] = -INFINITY;
                    mx = fmaxf(mx, s[i]);
                }
            }
            // the row's maximum over both halves
            xmax[(b * 2 + grp) * ROWS + R] = mx;
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(x_full(b));
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(x_full(b), (j >> 1) & 1, abort_flag))) { alive = false; break; }
            mx = fmaxf(mx, xmax[(b * 2 + (grp ^ 1)) * ROWS + R]);
            const float mn = fmaxf(m, mx);
            const float ref = mn == -INFINITY ? 0.f : mn;
            const float corr = expf(m - ref);             // exp(-inf) = 0 before the row's first visible key
            const bool rose = mn > m;
            m = mn;
            float sum = 0.f;
            uint32_t ph[KH / 2], pl[KH / 2];
#pragma unroll
            for (int i = 0; i < KH; i += 2) {
                // (the fast exponential: one special-function instruction per probability, relative error ~2^-21,
                // far inside what the f16 pair that follows keeps; the softmax threads are this kernel's critical path)
                const float x0 = __expf(s[i] - ref), x1 = __expf(s[i + 1] - ref);
                sum += x0 + x1;
                const __half2 hh = __floats2half2_rn(x0, x1);
                const float2 back = __half22float2(hh);
                ph[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                pl[i >> 1] = pack_half2(x0 - back.x, x1 - back.y);
            }
            l = l * corr + sum;                           // this half's share of the row's sum
            // O in tensor memory follows the new maximum: only when some row of the warp rose, and only once the
            // previous tile's P V has landed; each half takes half of O's columns
            if (j > 0 && __any_sync(0xffffffffu, rose)) {
                if (!__all_sync(0xffffffffu, tc5::mbar_wait(pv_done((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag))) { alive = false; break; }
                tc5::fence_after_sync();
#pragma unroll
                for (int c = 0; c < OH; c += 32) {
                    float v[16], w[16];
                    tc5::tmem_ld16x2(t_lane + TMEM_O + grp * OH + c, t_lane + TMEM_O + grp * OH + c + 16, v, w);
                    uint32_t o[32];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        o[i] = __float_as_uint(v[i] * corr);
                        o[16 + i] = __float_as_uint(w[i] * corr);
                    }
                    tc5::tmem_st32(t_lane + TMEM_O + grp * OH + c, o);
                }
            }
            // P buffer b was last read by the P V of tile j - 2
            if (!__all_sync(0xffffffffu, tc5::mbar_wait(pv_done(b), ((j >> 1) & 1) ^ 1, abort_flag))) { alive = false; break; }
            tc5::fence_after_sync();
            tc5::tmem_st16(t_lane + TMEM_P + b * 64 + grp * (KH / 2), ph);
            tc5::tmem_st16(t_lane + TMEM_P + b * 64 + 32 + grp * (KH / 2), pl);
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(p_full(b));
        }
        if (alive && n_tiles > 0 && __all_sync(0xffffffffu, tc5::mbar_wait(pv_done((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag))) {
            tc5::fence_after_sync();
            // the row's sum over both halves
            xsum[grp * ROWS + R] = l;
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(l_full);
            if (__all_sync(0xffffffffu, tc5::mbar_wait(l_full, 0, abort_flag))) {
                l += xsum[(grp ^ 1) * ROWS + R];
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                float * dst = out + (size_t)(i0 + (tt < ntok ? tt : 0)) * ldo + (size_t)(hk * G + hg) * HD + grp * OH;
#pragma unroll
                for (int c = 0; c < OH; c += 32) {
                    float v[16], w[16];
                    tc5::tmem_ld16x2(t_lane + TMEM_O + grp * OH + c, t_lane + TMEM_O + grp * OH + c + 16, v, w);
                    if (tt < ntok) {
#pragma unroll
                        for (int i = 0; i < 16; i += 4) {
                            *reinterpret_cast<float4 *>(dst + c + i) = make_float4(v[i] * inv, v[i + 1] * inv, v[i + 2] * inv, v[i + 3] * inv);
                            *reinterpret_cast<float4 *>(dst + c + 16 + i) = make_float4(w[i] * inv, w[i + 1] * inv, w[i + 2] * inv, w[i + 3] * inv);
                        }
                    }
                }
            }
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (tid == 0 && *abort_flag) atomicExch(error_flag, 1);
}

template <int HD>
void launch_hd(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const AttentionMaps & maps, const int2 * items, int n_items,
               const int32_t * tok_slot, const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int skip_small, int * error_flag,
               cudaStream_t stream) {
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) cudaFuncSetAttribute(attention_tc5_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<HD>::SMEM_BYTES);
    attention_tc5_kernel<HD><<<dim3(n_items, kv.n_head_kv), THREADS, Shape<HD>::SMEM_BYTES, stream>>>(qkv, ld, n_head, kv, layer, maps, items, tok_slot,
                                                                                                 tok_pos, tok_pos_min, out, ldo, skip_small, error_flag);
}

} // namespace

bool attention_tc5_supported(int n_head, int n_head_kv, int head_dim, int block_tokens, const AttentionMaps & maps) {
    const int G = n_head_kv ? n_head / n_head_kv : 0;
    return maps.valid && (head_dim == 64 || head_dim == 128) && block_tokens == 16 && n_head % n_head_kv == 0 &&
           (G == 1 || G == 2 || G == 4 || G == 8 || G == 16);
}

void launch_attention_tc5(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const AttentionMaps & maps, const int2 * items, int n_items,
                          const int32_t * tok_slot, const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, bool skip_small,
                          int * error_flag, cudaStream_t stream) {
    if (n_items <= 0) return;
    if (kv.head_dim == 128)
        launch_hd<128>(qkv, ld, n_head, kv, layer, maps, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, skip_small ? 1 : 0, error_flag, stream);
    else
        launch_hd<64>(qkv, ld, n_head, kv, layer, maps, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, skip_small ? 1 : 0, error_flag, stream);
}

} // namespace rb200
