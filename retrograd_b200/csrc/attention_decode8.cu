// Paged attention for work items with at most eight (token, query head of the group) pairs: the
// plain decode row of a model whose GQA group is at most eight. Such an item is bound by the HBM
// stream of its K/V blocks, so the kernel is arranged around instruction count per byte and bytes in
// flight:
//   - the KEYS are the M = 16 dimension of the MMA and the (token, head) pairs its N = 8 columns, so no
//     tensor-core work is spent on padding rows: S^T[key][col] = K[key][:] . q[col][:] with the query
//     fragments held in registers for the whole kernel, and O^T[d][col] = V^T[d][key] . P^T[key][col];
//     the probabilities move from accumulator layout to operand layout with two movmatrix each;
//   - every warp owns its 16-token blocks (w, w + 4, ...) and its own three-slot cp.async ring, so
//     warps never wait for each other inside the loop;
//   - a long sequence can be cut into `n_splits` block ranges handled by different CTAs (grid.z),
//     whose partial (max, sum, output) triples a second kernel merges: a step of a few sequences still
//     fills the GPU.
// Arithmetic as in attention_mma.cu: K and V exact f16 operands, query and probabilities as two-term
// f16 splits, f32 accumulation, online softmax per column.

#include "kernels.cuh"
#include "split_emit.cuh"
#include "mma_common.cuh"

#include <cfloat>

namespace rb200 {

namespace {

constexpr int D8_THREADS = 128;
constexpr int D8_SLOTS = 3;          // K/V blocks resident per warp
constexpr int D8_MAX_SPLITS = 16;    // CTAs sharing one item's KV blocks at most (the merge kernel holds that many triples in registers)

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
// 8x8 transpose of a matrix of b16 held one row per lane group (accumulator layout -> B operand layout)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

// partial results of one split: per column HD outputs (unnormalised), then max and sum
template <int HD>
__global__ void __launch_bounds__(D8_THREADS) attention_decode8_kernel(const float * __restrict__ qkv, int ld, int n_head, KvLayout kv, int layer,
                                                                        const int2 * __restrict__ items, const int32_t * __restrict__ tok_slot,
                                                                        const int32_t * __restrict__ tok_pos, const int32_t * __restrict__ tok_pos_min,
                                                                        float * __restrict__ out, int ldo, int n_splits, float * __restrict__ partial) {
    constexpr int PANELS = HD / 64;
    constexpr int KSTEPS = HD / 16;
    constexpr int MT = HD / 16;
    constexpr int TILE_BYTES = PANELS * 16 * 128;          // one K or V block
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_trigger();
    pdl_wait();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int hk = blockIdx.y, split = blockIdx.z;
    const int G = n_head / kv.n_head_kv;
    const int2 item = items[blockIdx.x];
    const int i0 = item.x, ntok = item.y;
    const int cols = ntok * G;
    if (cols > 8) return;                                   // served by the wider kernels
    const int slot = tok_slot[i0], pos0 = tok_pos[i0], pmin = tok_pos_min[i0];
    const int last = pos0 + ntok - 1;
    const int32_t * table = kv.block_table + (size_t)slot * kv.max_blocks;
    const __half * kbase = kv.k + layer * kv.layer_stride;
    const __half * vbase = kv.v + layer * kv.layer_stride;
    const float scale = rsqrtf((float)HD);

    const int nb0 = pmin >> 4, nb1 = last >> 4;
    const int n_blocks = nb1 - nb0 + 1;
    const int per = (n_blocks + n_splits - 1) / n_splits;
    const int b_lo = split * per, b_hi = min(n_blocks, b_lo + per);
    const int nw = b_hi > b_lo + warp ? (b_hi - b_lo - warp + 3) >> 2 : 0;      // this warp's blocks: b_lo + warp + 4 j

    uint8_t * ring = smem + (size_t)warp * D8_SLOTS * 2 * TILE_BYTES;
    auto load_block = [&](int j) {
        const int blk = rb_block(kv, table[nb0 + b_lo + warp + 4 * j]);
        const size_t base = ((size_t)blk * kv.n_head_kv + hk) * 16 * HD;
        const uint32_t k_s = smem_u32(ring + (j % D8_SLOTS) * 2 * TILE_BYTES), v_s = k_s + TILE_BYTES;
#pragma unroll
        for (int i = 0; i < 16 * HD / 8 / 32; ++i) {
            const int c = lane + i * 32;
            const int token = c / (HD / 8), dchunk = c % (HD / 8);
            const uint32_t off = (uint32_t)((dchunk >> 3) * (16 * 128)) + swz(token, dchunk & 7);
            cp_async16(k_s + off, kbase + base + (size_t)c * 8, 16);
            cp_async16(v_s + off, vbase + base + (size_t)c * 8, 16);
        }
    };
#pragma unroll
    for (int j = 0; j < D8_SLOTS - 1; ++j) {
        if (j < nw) load_block(j);
        cp_async_commit();
    }

    // ---- query fragments of column g = (token g / G, head g % G): B operand, K = the head dimension
    uint32_t qh[KSTEPS][2], ql[KSTEPS][2];
    {
        const bool valid = g < cols;
        const float * src = qkv + (size_t)(i0 + (valid ? g / G : 0)) * ld + (size_t)(hk * G + (valid ? g % G : 0)) * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                const float2 v = valid ? *reinterpret_cast<const float2 *>(src + ks * 16 + hlf * 8 + 2 * tq) : make_float2(0.f, 0.f);
                const float a = v.x * scale, b = v.y * scale;
                const __half2 hh = __floats2half2_rn(a, b);
                const float2 back = __half22float2(hh);
                qh[ks][hlf] = *reinterpret_cast<const uint32_t *>(&hh);
                ql[ks][hlf] = pack_h2(a - back.x, b - back.y);
            }
        }
    }
    // last visible position of this lane's two columns (2 tq, 2 tq + 1); -1 hides everything
    const int colA = 2 * tq, colB = 2 * tq + 1;
    const int prowA = colA < cols ? pos0 + colA / G : -1;
    const int prowB = colB < cols ? pos0 + colB / G : -1;

    float o[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

    for (int j = 0; j < nw; ++j) {
        cp_async_wait<D8_SLOTS - 2>();
        __syncwarp();                                      // block j has landed; every lane is done with block j - 1
        if (j + D8_SLOTS - 1 < nw) load_block(j + D8_SLOTS - 1);
        cp_async_commit();
        const uint32_t k_s = smem_u32(ring + (j % D8_SLOTS) * 2 * TILE_BYTES), v_s = k_s + TILE_BYTES;
        // S^T: rows = the block's 16 keys, columns = the (token, head) pairs
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a0, a1, a2, a3;
            const uint32_t off = (uint32_t)((ks >> 2) * (16 * 128)) + swz(lane & 15, (ks & 3) * 2 + (lane >> 4));
            ldmatrix_x4(k_s + off, a0, a1, a2, a3);
            mma_f16(s, a0, a1, a2, a3, qh[ks][0], qh[ks][1]);
            mma_f16(s2, a0, a1, a2, a3, ql[ks][0], ql[ks][1]);
        }
        const int p0 = ((nb0 + b_lo + warp + 4 * j) << 4) + g, p1 = p0 + 8;
        s[0] = (p0 < pmin || p0 > prowA) ? -INFINITY : s[0] + s2[0];
        s[1] = (p0 < pmin || p0 > prowB) ? -INFINITY : s[1] + s2[1];
        s[2] = (p1 < pmin || p1 > prowA) ? -INFINITY : s[2] + s2[2];
        s[3] = (p1 < pmin || p1 > prowB) ? -INFINITY : s[3] + s2[3];
        float mxA = fmaxf(s[0], s[2]), mxB = fmaxf(s[1], s[3]);
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) {
            mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, sh));
            mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, sh));
        }
        const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
        const float refA = mnA == -INFINITY ? 0.f : mnA, refB = mnB == -INFINITY ? 0.f : mnB;
        const float cA = expf(mA - refA), cB = expf(mB - refB);
        mA = mnA;
        mB = mnB;
        const float e0 = expf(s[0] - refA), e1 = expf(s[1] - refB), e2 = expf(s[2] - refA), e3 = expf(s[3] - refB);
        lA = lA * cA + (e0 + e2);
        lB = lB * cB + (e1 + e3);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            o[mt][0] *= cA;
            o[mt][1] *= cB;
            o[mt][2] *= cA;
            o[mt][3] *= cB;
        }
        // P^T as B operand (K = keys): accumulator rows (key g | g + 8) x columns (2 tq, 2 tq + 1) -> transpose
        const __half2 h01 = __floats2half2_rn(e0, e1), h23 = __floats2half2_rn(e2, e3);
        const float2 k01 = __half22float2(h01), k23 = __half22float2(h23);
        const uint32_t bh0 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&h01));
        const uint32_t bh1 = movmatrix_trans(*reinterpret_cast<const uint32_t *>(&h23));
        const uint32_t bl0 = movmatrix_trans(pack_h2(e0 - k01.x, e1 - k01.y));
        const uint32_t bl1 = movmatrix_trans(pack_h2(e2 - k23.x, e3 - k23.y));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            uint32_t a0, a1, a2, a3;
            const int chunk = mt * 2 + ((lane >> 3) & 1);
            const uint32_t off = (uint32_t)((chunk >> 3) * (16 * 128)) + swz((lane & 7) + ((lane >> 4) << 3), chunk & 7);
            ldmatrix_x4_trans(v_s + off, a0, a1, a2, a3);
            mma_f16(o[mt], a0, a1, a2, a3, bh0, bh1);
            mma_f16(o[mt], a0, a1, a2, a3, bl0, bl1);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
        lA += __shfl_xor_sync(0xffffffffu, lA, sh);
        lB += __shfl_xor_sync(0xffffffffu, lB, sh);
    }
    __syncthreads();                                        // every warp is done with its ring

    // ---- merge the four warps: per warp [8 columns][HD] outputs, then max and sum per column
    float * part_o = reinterpret_cast<float *>(smem);                       // [4][8][HD]
    float * part_m = part_o + 4 * 8 * HD;                                   // [4][8]
    float * part_l = part_m + 4 * 8;                                        // [4][8]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        float * dA = part_o + ((size_t)warp * 8 + colA) * HD + mt * 16 + g;
        float * dB = part_o + ((size_t)warp * 8 + colB) * HD + mt * 16 + g;
        dA[0] = o[mt][0];
        dB[0] = o[mt][1];
        dA[8] = o[mt][2];
        dB[8] = o[mt][3];
    }
    if (g == 0) {
        part_m[warp * 8 + colA] = mA;
        part_m[warp * 8 + colB] = mB;
        part_l[warp * 8 + colA] = lA;
        part_l[warp * 8 + colB] = lB;
    }
    __syncthreads();
    float * pdst = partial + (((size_t)blockIdx.x * kv.n_head_kv + hk) * n_splits + split) * 8 * (HD + 2);
    for (int idx = tid; idx < cols * HD; idx += D8_THREADS) {
        const int c = idx / HD, dcol = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, part_m[w * 8 + c]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = part_m[w * 8 + c];
            const float f = mw == -INFINITY ? 0.f : expf(mw - M);
            num += f * part_o[((size_t)w * 8 + c) * HD + dcol];
            den += f * part_l[w * 8 + c];
        }
        if (n_splits == 1) {
            out[(size_t)(i0 + c / G) * ldo + (size_t)(hk * G + c % G) * HD + dcol] = num / den;
        } else {
            pdst[(size_t)c * (HD + 2) + dcol] = num;
            if (dcol == 0) {
                pdst[(size_t)c * (HD + 2) + HD] = M;
                pdst[(size_t)c * (HD + 2) + HD + 1] = den;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same work over a Q8_0 pool, read as stored: half the bytes per key of the f16 pool, no dequantised copy.
// A pool row is [head_dim int8 | head_dim / 32 f16 scales] (kv_row_bytes); a block's 16 rows of K (or V) are one
// contiguous run that the warp copies into its ring as it is. The int8 quants are exact f16 operands, the scales are
// applied in f32:
//   - S^T: one accumulator per 32-element quant block (two K = 16 steps each), then s = sum_b scale[key][b] * acc_b.
//     The order of K inside an MMA step and of the keys among the MMA's rows is free as long as both operands agree,
//     so a lane reads eight consecutive quants of a block with one 64-bit load (word w feeds step w: bytes 0, 1 as the
//     k = 2 tq pair, bytes 2, 3 as the k = 2 tq + 8 pair) and MMA row m holds key pi(m) = 4 ((m & 7) >> 1) + (m & 1) +
//     2 (m >> 3), which makes the probabilities' B operand (after the transpose) carry keys 4 tq .. 4 tq + 3 - the four
//     V rows this lane reads;
//   - O^T: per 32-wide chunk of the head dimension (one quant block of V) the probabilities are scaled by that chunk's
//     scale of their key, split into two f16 terms and transposed; a lane reads one word (d = 4 g .. 4 g + 3 of the
//     chunk) from each of its four keys and pairs the bytes of two keys into the f16 pairs of two M tiles whose rows
//     are d = 4 g, 4 g + 1 (tile 2 c) and 4 g + 2, 4 g + 3 (tile 2 c + 1) - the merge below writes them back in order.
// int8 -> f16: (q ^ 0x80) is q + 128 as an unsigned byte and 0x6400 | byte the f16 value 1152 + q. V subtracts the 1152
// per element; K does not: its MMAs run on 1152 + q and the block's accumulator is corrected by 1152 times the sum of
// the query's (two-term) elements of that block, which a lane computes once for the two columns it accumulates.
// QBITS = 4, a Q4_0 pool (row = [head_dim / 2 bytes of nibble pairs | scales], value (q - 8) * scale, byte j of a
// block holding element j in its low and element j + 16 in its high nibble): the same scheme with other index maps. A
// lane's one word of a K block holds four low nibbles (step 2 b: elements 4 tq .. + 3) and four high ones (step
// 2 b + 1: elements 16 + 4 tq .. + 3); masked to bytes, 0x6400 | q is 1024 + q, so K runs on 1024 + q with the correction
// 1032 x the query sums, and V subtracts 1032. For V, lanes g and g + 4 read the same word of a key and take its low
// and its high nibbles: the lane's four values of the chunk are d = 16 (g >> 2) + 4 (g & 3) .. + 3.
template <int HD, int Q8_SLOTS, int MIN_CTAS, int QBITS>
__global__ void __launch_bounds__(D8_THREADS, MIN_CTAS) attention_decode8_q8_kernel(const float * __restrict__ qkv, int ld, int n_head, KvLayout kv, int layer,
                                                                           const int2 * __restrict__ items, const int32_t * __restrict__ tok_slot,
                                                                           const int32_t * __restrict__ tok_pos, const int32_t * __restrict__ tok_pos_min,
                                                                           float * __restrict__ out, int ldo, int n_splits, float * __restrict__ partial) {
    constexpr bool Q4 = QBITS == 4;
    constexpr int QBYTES = Q4 ? HD / 2 : HD;               // bytes of quants in a pool row; the scales follow
    constexpr int ROWB = (QBYTES + HD / 16 + 7) & ~7;      // bytes of a pool row (kv_row_bytes)
    constexpr float OFFSET = Q4 ? 1032.f : 1152.f;         // what 0x6400 | byte reads as, minus the quant's value
    constexpr int NB = HD / 32;                            // quant blocks per row
    constexpr int MT = HD / 16;
    constexpr int TILE_BYTES = 16 * ROWB;                  // one K or V block of one head
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_trigger();
    pdl_wait();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int hk = blockIdx.y, split = blockIdx.z;
    const int G = n_head / kv.n_head_kv;
    const int2 item = items[blockIdx.x];
    const int i0 = item.x, ntok = item.y;
    const int cols = ntok * G;
    if (cols > 8) return;                                   // served by the wider kernels
    const int slot = tok_slot[i0], pos0 = tok_pos[i0], pmin = tok_pos_min[i0];
    const int last = pos0 + ntok - 1;
    const int32_t * table = kv.block_table + (size_t)slot * kv.max_blocks;
    const uint8_t * kbase = kv.kq + layer * kv.q_layer_stride;
    const uint8_t * vbase = kv.vq + layer * kv.q_layer_stride;
    const float scale = rsqrtf((float)HD);

    const int nb0 = pmin >> 4, nb1 = last >> 4;
    const int n_blocks = nb1 - nb0 + 1;
    const int per = (n_blocks + n_splits - 1) / n_splits;
    const int b_lo = split * per, b_hi = min(n_blocks, b_lo + per);
    const int nw = b_hi > b_lo + warp ? (b_hi - b_lo - warp + 3) >> 2 : 0;      // this warp's blocks: b_lo + warp + 4 j

    uint8_t * ring = smem + (size_t)warp * Q8_SLOTS * 2 * TILE_BYTES;
    auto load_block = [&](int j) {
        const int blk = rb_block(kv, table[nb0 + b_lo + warp + 4 * j]);
        const size_t base = ((size_t)blk * kv.n_head_kv + hk) * TILE_BYTES;
        const uint32_t k_s = smem_u32(ring + (j % Q8_SLOTS) * 2 * TILE_BYTES), v_s = k_s + TILE_BYTES;
        for (int c = lane; c < TILE_BYTES / 16; c += 32) {
            cp_async16(k_s + c * 16, kbase + base + (size_t)c * 16, 16);
            cp_async16(v_s + c * 16, vbase + base + (size_t)c * 16, 16);
        }
    };
#pragma unroll
    for (int j = 0; j < Q8_SLOTS - 1; ++j) {
        if (j < nw) load_block(j);
        cp_async_commit();
    }

    // ---- query fragments of column g = (token g / G, head g % G): step 2 b + w holds elements 32 b + 8 tq + 4 w .. + 3
    uint32_t qh[2 * NB][2], ql[2 * NB][2];
    {
        const bool valid = g < cols;
        const float * src = qkv + (size_t)(i0 + (valid ? g / G : 0)) * ld + (size_t)(hk * G + (valid ? g % G : 0)) * HD;
#pragma unroll
        for (int ks = 0; ks < 2 * NB; ++ks) {
            const int e0 = Q4 ? (ks >> 1) * 32 + 16 * (ks & 1) + 4 * tq : (ks >> 1) * 32 + 8 * tq + 4 * (ks & 1);
            const float4 v = valid ? *reinterpret_cast<const float4 *>(src + e0) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float e[4] = {v.x * scale, v.y * scale, v.z * scale, v.w * scale};
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                const __half2 hh = __floats2half2_rn(e[2 * hlf], e[2 * hlf + 1]);
                const float2 back = __half22float2(hh);
                qh[ks][hlf] = *reinterpret_cast<const uint32_t *>(&hh);
                ql[ks][hlf] = pack_h2(e[2 * hlf] - back.x, e[2 * hlf + 1] - back.y);
            }
        }
    }
    const int colA = 2 * tq, colB = 2 * tq + 1;
    const int prowA = colA < cols ? pos0 + colA / G : -1;
    const int prowB = colB < cols ? pos0 + colB / G : -1;
    const int key0 = 4 * (g >> 1) + (g & 1), key1 = key0 + 2;      // the keys of this lane's accumulator rows g and g + 8
    // 1152 x the sum over quant block b of the query terms, for this lane's accumulator columns 2 tq and 2 tq + 1
    float corrA[NB], corrB[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 2; ++w) {
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&qh[2 * b + w][hlf]));
                const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&ql[2 * b + w][hlf]));
                sum += (a.x + c.x) + (a.y + c.y);
            }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);       // the four lanes of column g hold the block's 32 elements
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        corrA[b] = OFFSET * __shfl_sync(0xffffffffu, sum, colA * 4);
        corrB[b] = OFFSET * __shfl_sync(0xffffffffu, sum, colB * 4);
    }
    auto raw_lo = [](uint32_t w) { return __byte_perm(w, 0x64646464u, 0x4140); };     // f16 pair (1152 + q) of bytes 0, 1
    auto raw_hi = [](uint32_t w) { return __byte_perm(w, 0x64646464u, 0x4342); };     // ... of bytes 2, 3
    const __half2 bias2 = __floats2half2_rn(OFFSET, OFFSET);
    auto pair_lo = [&](uint32_t w) { const uint32_t t = __byte_perm(w, 0x64646464u, 0x4140); return __hsub2(*reinterpret_cast<const __half2 *>(&t), bias2); };
    auto pair_hi = [&](uint32_t w) { const uint32_t t = __byte_perm(w, 0x64646464u, 0x4342); return __hsub2(*reinterpret_cast<const __half2 *>(&t), bias2); };
    auto as_u32 = [](__half2 h) { return *reinterpret_cast<const uint32_t *>(&h); };

    float o[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

    for (int j = 0; j < nw; ++j) {
        cp_async_wait<Q8_SLOTS - 2>();
        __syncwarp();                                      // block j has landed; every lane is done with block j - 1
        if (j + Q8_SLOTS - 1 < nw) load_block(j + Q8_SLOTS - 1);
        cp_async_commit();
        const uint8_t * k_s = ring + (j % Q8_SLOTS) * 2 * TILE_BYTES, * v_s = k_s + TILE_BYTES;
        // S^T: rows = keys (key0 | key1), columns = the (token, head) pairs; per quant block, then scaled
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        const __half * ks0 = reinterpret_cast<const __half *>(k_s + key0 * ROWB + QBYTES), * ks1 = reinterpret_cast<const __half *>(k_s + key1 * ROWB + QBYTES);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            uint2 r0, r1;       // .x: the bytes of step 2 b, .y: of step 2 b + 1; rows key0 and key1
            if (Q4) {
                const uint32_t w0 = *reinterpret_cast<const uint32_t *>(k_s + key0 * ROWB + b * 16 + 4 * tq);
                const uint32_t w1 = *reinterpret_cast<const uint32_t *>(k_s + key1 * ROWB + b * 16 + 4 * tq);
                r0 = make_uint2(w0 & 0x0F0F0F0Fu, (w0 >> 4) & 0x0F0F0F0Fu);
                r1 = make_uint2(w1 & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu);
            } else {
                r0 = *reinterpret_cast<const uint2 *>(k_s + key0 * ROWB + b * 32 + 8 * tq);
                r1 = *reinterpret_cast<const uint2 *>(k_s + key1 * ROWB + b * 32 + 8 * tq);
                r0.x ^= 0x80808080u; r0.y ^= 0x80808080u; r1.x ^= 0x80808080u; r1.y ^= 0x80808080u;
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const uint32_t a0 = raw_lo(r0.x), a1 = raw_lo(r1.x), a2 = raw_hi(r0.x), a3 = raw_hi(r1.x);
                mma_f16(acc, a0, a1, a2, a3, qh[2 * b][0], qh[2 * b][1]);
                mma_f16(acc, a0, a1, a2, a3, ql[2 * b][0], ql[2 * b][1]);
            }
            {
                const uint32_t a0 = raw_lo(r0.y), a1 = raw_lo(r1.y), a2 = raw_hi(r0.y), a3 = raw_hi(r1.y);
                mma_f16(acc, a0, a1, a2, a3, qh[2 * b + 1][0], qh[2 * b + 1][1]);
                mma_f16(acc, a0, a1, a2, a3, ql[2 * b + 1][0], ql[2 * b + 1][1]);
            }
            const float d0 = __half2float(ks0[b]), d1 = __half2float(ks1[b]);
            s[0] += d0 * (acc[0] - corrA[b]);
            s[1] += d0 * (acc[1] - corrB[b]);
            s[2] += d1 * (acc[2] - corrA[b]);
            s[3] += d1 * (acc[3] - corrB[b]);
        }
        const int p0 = ((nb0 + b_lo + warp + 4 * j) << 4) + key0, p1 = p0 + 2;
        s[0] = (p0 < pmin || p0 > prowA) ? -INFINITY : s[0];
        s[1] = (p0 < pmin || p0 > prowB) ? -INFINITY : s[1];
        s[2] = (p1 < pmin || p1 > prowA) ? -INFINITY : s[2];
        s[3] = (p1 < pmin || p1 > prowB) ? -INFINITY : s[3];
        float mxA = fmaxf(s[0], s[2]), mxB = fmaxf(s[1], s[3]);
#pragma unroll
        for (int sh = 4; sh < 32; sh <<= 1) {
            mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, sh));
            mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, sh));
        }
        const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
        const float refA = mnA == -INFINITY ? 0.f : mnA, refB = mnB == -INFINITY ? 0.f : mnB;
        // (this kernel is bound by instruction issue: the one-instruction exponential, relative error ~2^-21 and far inside
        // what the two-term f16 probabilities keep, and no rescale of O while no column's maximum moves)
        const bool moved = mnA != mA || mnB != mB;
        const float cA = __expf(mA - refA), cB = __expf(mB - refB);
        mA = mnA;
        mB = mnB;
        const float e0 = __expf(s[0] - refA), e1 = __expf(s[1] - refB), e2 = __expf(s[2] - refA), e3 = __expf(s[3] - refB);
        lA = lA * cA + (e0 + e2);
        lB = lB * cB + (e1 + e3);
        if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                o[mt][0] *= cA;
                o[mt][1] *= cB;
                o[mt][2] *= cA;
                o[mt][3] *= cB;
            }
        }
        const __half * vs0 = reinterpret_cast<const __half *>(v_s + key0 * ROWB + QBYTES), * vs1 = reinterpret_cast<const __half *>(v_s + key1 * ROWB + QBYTES);
#pragma unroll
        for (int c = 0; c < NB; ++c) {
            // the probabilities times this chunk's V scale of their key, as two f16 terms, transposed into B operands
            const float d0 = __half2float(vs0[c]), d1 = __half2float(vs1[c]);
            const float f0 = e0 * d0, f1 = e1 * d0, f2 = e2 * d1, f3 = e3 * d1;
            const __half2 h01 = __floats2half2_rn(f0, f1), h23 = __floats2half2_rn(f2, f3);
            const float2 k01 = __half22float2(h01), k23 = __half22float2(h23);
            const uint32_t bh0 = movmatrix_trans(as_u32(h01)), bh1 = movmatrix_trans(as_u32(h23));
            const uint32_t bl0 = movmatrix_trans(pack_h2(f0 - k01.x, f1 - k01.y)), bl1 = movmatrix_trans(pack_h2(f2 - k23.x, f3 - k23.y));
            // V words of keys 4 tq .. 4 tq + 3: four bytes (Q8_0: d = 32 c + 4 g .. + 3; Q4_0: the low or high nibbles of
            // bytes 4 (g & 3) .. + 3 of the chunk, d = 32 c + 16 (g >> 2) + 4 (g & 3) .. + 3), each byte 0x6400-ready
            uint32_t w0, w1, w2, w3;
            if (Q4) {
                const uint8_t * vrow = v_s + (4 * tq) * ROWB + c * 16 + 4 * (g & 3);
                const int sh = 4 * (g >> 2);
                w0 = (*reinterpret_cast<const uint32_t *>(vrow) >> sh) & 0x0F0F0F0Fu;
                w1 = (*reinterpret_cast<const uint32_t *>(vrow + ROWB) >> sh) & 0x0F0F0F0Fu;
                w2 = (*reinterpret_cast<const uint32_t *>(vrow + 2 * ROWB) >> sh) & 0x0F0F0F0Fu;
                w3 = (*reinterpret_cast<const uint32_t *>(vrow + 3 * ROWB) >> sh) & 0x0F0F0F0Fu;
            } else {
                const uint8_t * vrow = v_s + (4 * tq) * ROWB + c * 32 + 4 * g;
                w0 = *reinterpret_cast<const uint32_t *>(vrow) ^ 0x80808080u;
                w1 = *reinterpret_cast<const uint32_t *>(vrow + ROWB) ^ 0x80808080u;
                w2 = *reinterpret_cast<const uint32_t *>(vrow + 2 * ROWB) ^ 0x80808080u;
                w3 = *reinterpret_cast<const uint32_t *>(vrow + 3 * ROWB) ^ 0x80808080u;
            }
            // (key 4 tq, key 4 tq + 1) byte pairs of d offsets 0, 1 | 2, 3; the same for keys 4 tq + 2, 4 tq + 3
            const uint32_t u01 = __byte_perm(w0, w1, 0x5140), u23 = __byte_perm(w0, w1, 0x7362);
            const uint32_t x01 = __byte_perm(w2, w3, 0x5140), x23 = __byte_perm(w2, w3, 0x7362);
            {
                const uint32_t a0 = as_u32(pair_lo(u01)), a1 = as_u32(pair_hi(u01)), a2 = as_u32(pair_lo(x01)), a3 = as_u32(pair_hi(x01));
                mma_f16(o[2 * c], a0, a1, a2, a3, bh0, bh1);
                mma_f16(o[2 * c], a0, a1, a2, a3, bl0, bl1);
            }
            {
                const uint32_t a0 = as_u32(pair_lo(u23)), a1 = as_u32(pair_hi(u23)), a2 = as_u32(pair_lo(x23)), a3 = as_u32(pair_hi(x23));
                mma_f16(o[2 * c + 1], a0, a1, a2, a3, bh0, bh1);
                mma_f16(o[2 * c + 1], a0, a1, a2, a3, bl0, bl1);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
        lA += __shfl_xor_sync(0xffffffffu, lA, sh);
        lB += __shfl_xor_sync(0xffffffffu, lB, sh);
    }
    __syncthreads();                                        // every warp is done with its ring

    // ---- merge the four warps: per warp [8 columns][HD] outputs, then max and sum per column
    float * part_o = reinterpret_cast<float *>(smem);                       // [4][8][HD]
    float * part_m = part_o + 4 * 8 * HD;                                   // [4][8]
    float * part_l = part_m + 4 * 8;                                        // [4][8]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        // M tile mt = 2 c + y: accumulator row g is d = 32 c + (the lane's first d of the chunk) + 2 y, row g + 8 is d + 1
        const int d = 32 * (mt >> 1) + (Q4 ? 16 * (g >> 2) + 4 * (g & 3) : 4 * g) + 2 * (mt & 1);
        float * dA = part_o + ((size_t)warp * 8 + colA) * HD + d;
        float * dB = part_o + ((size_t)warp * 8 + colB) * HD + d;
        dA[0] = o[mt][0];
        dB[0] = o[mt][1];
        dA[1] = o[mt][2];
        dB[1] = o[mt][3];
    }
    if (g == 0) {
        part_m[warp * 8 + colA] = mA;
        part_m[warp * 8 + colB] = mB;
        part_l[warp * 8 + colA] = lA;
        part_l[warp * 8 + colB] = lB;
    }
    __syncthreads();
    float * pdst = partial + (((size_t)blockIdx.x * kv.n_head_kv + hk) * n_splits + split) * 8 * (HD + 2);
    for (int idx = tid; idx < cols * HD; idx += D8_THREADS) {
        const int c = idx / HD, dcol = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, part_m[w * 8 + c]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = part_m[w * 8 + c];
            const float f = mw == -INFINITY ? 0.f : expf(mw - M);
            num += f * part_o[((size_t)w * 8 + c) * HD + dcol];
            den += f * part_l[w * 8 + c];
        }
        if (n_splits == 1) {
            out[(size_t)(i0 + c / G) * ldo + (size_t)(hk * G + c % G) * HD + dcol] = num / den;
        } else {
            pdst[(size_t)c * (HD + 2) + dcol] = num;
            if (dcol == 0) {
                pdst[(size_t)c * (HD + 2) + HD] = M;
                pdst[(size_t)c * (HD + 2) + HD + 1] = den;
            }
        }
    }
}

// out = merge over the splits of one (item, kv head, column): grid (items, kv heads, 8), HD threads
template <int HD>
__global__ void attention_decode8_merge_kernel(const float * __restrict__ partial, int n_head, int n_head_kv, const int2 * __restrict__ items,
                                               float * __restrict__ out, int ldo, int n_splits, SplitAct split) {
    pdl_trigger();
    pdl_wait();
    const int G = n_head / n_head_kv;
    const int2 item = items[blockIdx.x];
    const int cols = item.y * G, c = blockIdx.z;
    if (cols > 8 || c >= cols) return;
    const int hk = blockIdx.y, dcol = threadIdx.x;
    const float * src = partial + (((size_t)blockIdx.x * n_head_kv + hk) * n_splits * 8 + c) * (HD + 2);
    // every split's (max, sum, value) is loaded before the first use: one memory latency, not one per split
    float mz[D8_MAX_SPLITS], lz[D8_MAX_SPLITS], vz[D8_MAX_SPLITS];
#pragma unroll
    for (int z = 0; z < D8_MAX_SPLITS; ++z) {
        const float * p = src + (size_t)z * 8 * (HD + 2);
        const bool on = z < n_splits;
        mz[z] = on ? p[HD] : -INFINITY;
        lz[z] = on ? p[HD + 1] : 0.f;
        vz[z] = on ? p[dcol] : 0.f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int z = 0; z < D8_MAX_SPLITS; ++z) M = fmaxf(M, mz[z]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int z = 0; z < D8_MAX_SPLITS; ++z) {
        if (z < n_splits) {
            const float f = mz[z] == -INFINITY ? 0.f : expf(mz[z] - M);
            num += f * vz[z];
            den += f * lz[z];
        }
    }
    const float v = num / den;
    const int row = item.x + c / G, col = (hk * G + c % G) * HD + dcol;
    out[(size_t)row * ldo + col] = v;
    // a warp covers one 32-column sub-block of the head: the split form the output projection reads
    if (split.hi) emit_split(split, row, col, v);
}

template <int HD>
void launch_hd8(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items, const int32_t * tok_slot,
                const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int n_splits, float * scratch, cudaStream_t stream,
                const SplitAct & split) {
    constexpr int smem = 4 * D8_SLOTS * 2 * (HD / 64) * 16 * 128;
    static_assert(smem >= (4 * 8 * HD + 64) * 4, "the merge buffers fit the K/V rings");
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) cudaFuncSetAttribute(attention_decode8_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (kv.storage == KV_Q8_0) {
        // three ring slots and four CTAs per SM (128 registers): two slots with five or six CTAs (96 / 80 registers, spills)
        // measured 7 % and 20 % slower on the ragged 256-request workload
        constexpr int smem_q8 = 4 * D8_SLOTS * 2 * 16 * ((HD + HD / 16 + 7) & ~7);
        static_assert(smem_q8 >= (4 * 8 * HD + 64) * 4, "the merge buffers fit the quantised K/V rings");
        static PerDeviceOnce once;
        if (once.first()) cudaFuncSetAttribute(attention_decode8_q8_kernel<HD, D8_SLOTS, 4, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q8);
        launch_pdl(attention_decode8_q8_kernel<HD, D8_SLOTS, 4, 8>, dim3(n_items, kv.n_head_kv, n_splits), dim3(D8_THREADS), smem_q8, stream, qkv, ld, n_head,
                   kv, layer, items, tok_slot, tok_pos, tok_pos_min, out, ldo, n_splits, scratch);
    } else if (kv.storage == KV_Q4_0) {
        // the ring holds as many blocks as fit the merge buffers' bytes (a Q4_0 block of K and V is 2.3 KB at head_dim 128)
        constexpr int tile = 16 * ((HD / 2 + HD / 16 + 7) & ~7);
        constexpr int slots = (4 * 8 * HD + 64) * 4 > 4 * D8_SLOTS * 2 * tile ? ((4 * 8 * HD + 64) * 4 + 4 * 2 * tile - 1) / (4 * 2 * tile) : D8_SLOTS;
        constexpr int smem_q4 = 4 * slots * 2 * tile;
        static_assert(smem_q4 >= (4 * 8 * HD + 64) * 4, "the merge buffers fit the quantised K/V rings");
        static PerDeviceOnce once;
        if (once.first()) cudaFuncSetAttribute(attention_decode8_q8_kernel<HD, slots, 4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q4);
        launch_pdl(attention_decode8_q8_kernel<HD, slots, 4, 4>, dim3(n_items, kv.n_head_kv, n_splits), dim3(D8_THREADS), smem_q4, stream, qkv, ld, n_head,
                   kv, layer, items, tok_slot, tok_pos, tok_pos_min, out, ldo, n_splits, scratch);
    } else
        launch_pdl(attention_decode8_kernel<HD>, dim3(n_items, kv.n_head_kv, n_splits), dim3(D8_THREADS), smem, stream, qkv, ld, n_head, kv, layer, items,
                   tok_slot, tok_pos, tok_pos_min, out, ldo, n_splits, scratch);
    if (n_splits > 1)
        launch_pdl(attention_decode8_merge_kernel<HD>, dim3(n_items, kv.n_head_kv, 8), dim3(HD), 0, stream, scratch, n_head, kv.n_head_kv, items, out,
                   ldo, n_splits, split);
}

} // namespace

bool attention_decode8_supported(int n_head, int n_head_kv, int head_dim, int block_tokens) {
    return (head_dim == 64 || head_dim == 128) && block_tokens == 16 && n_head % n_head_kv == 0 && n_head / n_head_kv <= 8;
}

int attention_decode8_max_splits() { return D8_MAX_SPLITS; }

size_t attention_decode8_scratch_floats(int n_items, int n_head_kv, int n_splits, int head_dim) {
    return n_splits > 1 ? (size_t)n_items * n_head_kv * n_splits * 8 * (head_dim + 2) : 0;
}

void launch_attention_decode8(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items,
                              const int32_t * tok_slot, const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int n_splits,
                              float * scratch, cudaStream_t stream, const SplitAct * split) {
    if (n_items <= 0) return;
    if (n_splits > D8_MAX_SPLITS) n_splits = D8_MAX_SPLITS;      // callers size the scratch with attention_decode8_max_splits()
    const SplitAct sa = split && n_splits > 1 ? *split : SplitAct{};
    if (kv.head_dim == 128)
        launch_hd8<128>(qkv, ld, n_head, kv, layer, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, n_splits, scratch, stream, sa);
    else
        launch_hd8<64>(qkv, ld, n_head, kv, layer, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, n_splits, scratch, stream, sa);
}

} // namespace rb200
