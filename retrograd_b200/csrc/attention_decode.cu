// Paged attention for work items whose query tile fits one m16 MMA tile (at most 16 query vectors:
// decode rows, and the ragged tail of a prefill chunk). Such an item is bound by the HBM stream of its
// K/V blocks, so the four warps of the CTA do not share blocks: warp w takes blocks w, w+4, w+8, ...
// of the slot, each under its own online softmax over the same 16 query rows, and the four partial
// results (max, sum, output) are merged through shared memory at the end. Twelve 16-token blocks
// (three rounds of four) are in flight per CTA through a cp.async ring, 96 KB of K/V.
//
// Arithmetic is the same as attention_mma.cu: K and V exact f16 operands, query and probabilities
// as two-term splits, f32 accumulation.

#include "kernels.cuh"
#include "mma_common.cuh"

#include <cfloat>

namespace rb200 {

namespace {

constexpr int DEC_THREADS = 128;
constexpr int DEC_ROUNDS = 3;                    // rounds of four blocks resident in shared memory

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(const float * __restrict__ qkv, int ld, int n_head, KvLayout kv, int layer,
                                                                       const int2 * __restrict__ items, const int32_t * __restrict__ tok_slot,
                                                                       const int32_t * __restrict__ tok_pos, const int32_t * __restrict__ tok_pos_min,
                                                                       float * __restrict__ out, int ldo, int min_cols) {
    constexpr int PANELS = HD / 64;
    constexpr int KSTEPS = HD / 16;
    constexpr int NT = HD / 8;
    constexpr int Q_BYTES = PANELS * 16 * 128;             // 16 query rows
    constexpr int TILE_BYTES = PANELS * 16 * 128;          // one K or V block
    constexpr int SLOTS = DEC_ROUNDS * 4;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t * q_hi = smem;
    uint8_t * q_lo = smem + Q_BYTES;
    uint8_t * kv_s = smem + 2 * Q_BYTES;                    // [slot][K | V]; reused for the merge at the end

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int hk = blockIdx.y;
    const int G = n_head / kv.n_head_kv;
    const int2 item = items[blockIdx.x];
    const int i0 = item.x, ntok = item.y;
    if (ntok * G > 16 || ntok * G <= min_cols) return;      // served by the tile kernel / the eight-column kernel
    const int slot = tok_slot[i0], pos0 = tok_pos[i0], pmin = tok_pos_min[i0];
    const int last = pos0 + ntok - 1;
    const int32_t * table = kv.block_table + (size_t)slot * kv.max_blocks;
    const __half * kbase = kv.k + layer * kv.layer_stride;
    const __half * vbase = kv.v + layer * kv.layer_stride;
    const float scale = rsqrtf((float)HD);

    // ---- the 16 query rows (token, head-in-group) as hi + lo f16: 8 threads per row
    {
        const int R = tid >> 3, part = tid & 7;             // row 0..15, eighth of the row
        const int tt = R / G, hg = R % G;
        const bool valid = tt < ntok;
        const float * src = qkv + (size_t)(i0 + (valid ? tt : 0)) * ld + (size_t)(hk * G + hg) * HD;
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
            const int col_chunk = part * (HD / 64) + c;     // 16-byte chunk (8 columns) of the row
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = valid ? src[col_chunk * 8 + e] * scale : 0.f;
            uint32_t h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __half2 hh = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                const float2 back = __half22float2(hh);
                h[e] = *reinterpret_cast<const uint32_t *>(&hh);
                l[e] = pack2(v[2 * e] - back.x, v[2 * e + 1] - back.y);
            }
            const uint32_t off = (uint32_t)((col_chunk >> 3) * (16 * 128)) + swz(R, col_chunk & 7);
            *reinterpret_cast<uint4 *>(q_hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4 *>(q_lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
        }
    }

    const int nb0 = pmin >> 4, nb1 = last >> 4;
    const int n_blocks = nb1 - nb0 + 1;
    const int n_rounds = (n_blocks + 3) >> 2;
    // every thread copies its share of each of the round's four blocks
    auto load_round = [&](int r) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int bi = r * 4 + w;
            if (bi < n_blocks) {
                const int blk = rb_block(kv, table[nb0 + bi]);
                const size_t base = ((size_t)blk * kv.n_head_kv + hk) * 16 * HD;
                const uint32_t k_s = smem_u32(kv_s + ((r % DEC_ROUNDS) * 4 + w) * 2 * TILE_BYTES);
                const uint32_t v_s = k_s + TILE_BYTES;
#pragma unroll
                for (int i = 0; i < 16 * HD / 8 / DEC_THREADS; ++i) {
                    const int c = tid + i * DEC_THREADS;
                    const int token = c / (HD / 8), dchunk = c % (HD / 8);
                    const uint32_t off = (uint32_t)((dchunk >> 3) * (16 * 128)) + swz(token, dchunk & 7);
                    cp_async16(k_s + off, kbase + base + (size_t)c * 8, 16);
                    cp_async16(v_s + off, vbase + base + (size_t)c * 8, 16);
                }
            }
        }
    };
#pragma unroll
    for (int r = 0; r < DEC_ROUNDS - 1; ++r) {
        if (r < n_rounds) load_round(r);
        cp_async_commit();
    }
    __syncthreads();

    uint32_t qh[KSTEPS][4], ql[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const uint32_t off = (uint32_t)((ks >> 2) * (16 * 128)) + swz(lane & 15, (ks & 3) * 2 + (lane >> 4));
        ldmatrix_x4(smem_u32(q_hi) + off, qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3]);
        ldmatrix_x4(smem_u32(q_lo) + off, ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3]);
    }

    const int tt0 = g / G, tt1 = (g + 8) / G;
    const int prow0 = tt0 < ntok ? pos0 + tt0 : -1;
    const int prow1 = tt1 < ntok ? pos0 + tt1 : -1;

    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int r = 0; r < n_rounds; ++r) {
        cp_async_wait<DEC_ROUNDS - 2>();
        __syncthreads();
        if (r + DEC_ROUNDS - 1 < n_rounds) load_round(r + DEC_ROUNDS - 1);
        cp_async_commit();
        const int bi = r * 4 + warp;
        if (bi >= n_blocks) continue;
        const uint32_t k_s = smem_u32(kv_s + ((r % DEC_ROUNDS) * 4 + warp) * 2 * TILE_BYTES);
        const uint32_t v_s = k_s + TILE_BYTES;
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t b0, b1, b2, b3;
            const uint32_t off = (uint32_t)((ks >> 2) * (16 * 128)) + swz((lane & 7) + ((lane >> 4) << 3), (ks & 3) * 2 + ((lane >> 3) & 1));
            ldmatrix_x4(k_s + off, b0, b1, b2, b3);
            mma_f16(s[0], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b0, b1);
            mma_f16(s[1], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b2, b3);
            mma_f16(s[0], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b0, b1);
            mma_f16(s[1], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b2, b3);
        }
        const int pbase = (nb0 + bi) << 4;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int p = pbase + ni * 8 + 2 * tq + e;
                if (p < pmin || p > prow0) s[ni][e] = -INFINITY;
                if (p < pmin || p > prow1) s[ni][2 + e] = -INFINITY;
                mx0 = fmaxf(mx0, s[ni][e]);
                mx1 = fmaxf(mx1, s[ni][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = expf(m0 - ref0), c1 = expf(m1 - ref1);
        m0 = mn0;
        m1 = mn1;
        float p[2][4];
        float add0 = 0.f, add1 = 0.f;
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
            p[ni][0] = expf(s[ni][0] - ref0);
            p[ni][1] = expf(s[ni][1] - ref0);
            p[ni][2] = expf(s[ni][2] - ref1);
            p[ni][3] = expf(s[ni][3] - ref1);
            add0 += p[ni][0] + p[ni][1];
            add1 += p[ni][2] + p[ni][3];
        }
        l0 = l0 * c0 + add0;
        l1 = l1 * c1 + add1;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            o[nt][0] *= c0;
            o[nt][1] *= c0;
            o[nt][2] *= c1;
            o[nt][3] *= c1;
        }
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int f = 0; f < 4; ++f) {
            const float x0 = p[f >> 1][(f & 1) * 2], x1 = p[f >> 1][(f & 1) * 2 + 1];
            const __half2 hh = __floats2half2_rn(x0, x1);
            const float2 back = __half22float2(hh);
            ph[f] = *reinterpret_cast<const uint32_t *>(&hh);
            pl[f] = pack2(x0 - back.x, x1 - back.y);
        }
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            uint32_t v0, v1, v2, v3;
            const uint32_t off = (uint32_t)((dp >> 2) * (16 * 128)) + swz((lane & 7) + (((lane >> 3) & 1) << 3), (dp & 3) * 2 + (lane >> 4));
            ldmatrix_x4_trans(v_s + off, v0, v1, v2, v3);
            mma_f16(o[2 * dp], ph[0], ph[1], ph[2], ph[3], v0, v1);
            mma_f16(o[2 * dp + 1], ph[0], ph[1], ph[2], ph[3], v2, v3);
            mma_f16(o[2 * dp], pl[0], pl[1], pl[2], pl[3], v0, v1);
            mma_f16(o[2 * dp + 1], pl[0], pl[1], pl[2], pl[3], v2, v3);
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();                                        // every warp is done with the K/V ring

    // ---- merge the four warps' partial results: per warp [16 rows][HD] outputs, then max and sum per row
    float * part_o = reinterpret_cast<float *>(kv_s);                       // [4][16][HD]
    float * part_m = part_o + 4 * 16 * HD;                                  // [4][16]
    float * part_l = part_m + 4 * 16;                                       // [4][16]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        float * d0 = part_o + ((size_t)warp * 16 + g) * HD + nt * 8 + 2 * tq;
        float * d1 = part_o + ((size_t)warp * 16 + g + 8) * HD + nt * 8 + 2 * tq;
        d0[0] = o[nt][0];
        d0[1] = o[nt][1];
        d1[0] = o[nt][2];
        d1[1] = o[nt][3];
    }
    if (tq == 0) {
        part_m[warp * 16 + g] = m0;
        part_m[warp * 16 + g + 8] = m1;
        part_l[warp * 16 + g] = l0;
        part_l[warp * 16 + g + 8] = l1;
    }
    __syncthreads();
    const int n_rows = ntok * G;
    for (int idx = tid; idx < n_rows * HD; idx += DEC_THREADS) {
        const int R = idx / HD, dcol = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, part_m[w * 16 + R]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = part_m[w * 16 + R];
            const float f = mw == -INFINITY ? 0.f : expf(mw - M);
            num += f * part_o[((size_t)w * 16 + R) * HD + dcol];
            den += f * part_l[w * 16 + R];
        }
        const int tt = R / G, hg = R % G;
        out[(size_t)(i0 + tt) * ldo + (size_t)(hk * G + hg) * HD + dcol] = num / den;
    }
}

template <int HD>
void launch_hd(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items, const int32_t * tok_slot,
               const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int min_cols, cudaStream_t stream) {
    constexpr int smem = 2 * (HD / 64) * 16 * 128 + DEC_ROUNDS * 4 * 2 * (HD / 64) * 16 * 128;
    static_assert(DEC_ROUNDS * 4 * 2 * (HD / 64) * 16 * 128 >= (4 * 16 * HD + 128) * 4, "the merge buffers fit the K/V ring");
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    attention_decode_kernel<HD><<<dim3(n_items, kv.n_head_kv), DEC_THREADS, smem, stream>>>(qkv, ld, n_head, kv, layer, items, tok_slot, tok_pos,
                                                                                          tok_pos_min, out, ldo, min_cols);
}

} // namespace

void launch_attention_decode(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items,
                             const int32_t * tok_slot, const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int min_cols,
                             cudaStream_t stream) {
    if (n_items <= 0) return;
    if (kv.head_dim == 128) launch_hd<128>(qkv, ld, n_head, kv, layer, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, min_cols, stream);
    else launch_hd<64>(qkv, ld, n_head, kv, layer, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, min_cols, stream);
}

} // namespace rb200
