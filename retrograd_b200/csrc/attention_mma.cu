// Paged attention over ragged sequences on the tensor cores: decode rows (one token) and prefill
// chunk rows (many tokens) in one launch.
//
// A CTA serves one work item = (up to 128 / G consecutive tokens of one step row) x (one KV head),
// G = query heads per KV head. Its 128 query vectors (token, head-in-group) form eight m16 tiles,
// one per warp (the wider the tile, the fewer times a prefill chunk re-reads its context). The KV blocks of the slot are found through the block table and streamed, 16
// tokens at a time, into a four-stage cp.async ring of 128B-swizzled shared-memory tiles that all
// eight warps share; scores and the output are accumulated with mma.sync m16n8k16 (f16 operands,
// f32 accumulators) under a warp-level online softmax.
//
// Accuracy: K and V are f16 by storage, so they are exact operands. The query (pre-scaled by
// 1/sqrt(head_dim)) and the probabilities are fed as two-term splits hi + lo, which keeps every
// product exact in f32; a single f16 rounding of q or p would cost ~3e-4 relative error per layer.
// Attention is bound by the HBM stream of K/V for decode rows, so the doubled MMA count is free
// there.

#include "kernels.cuh"
#include "mma_common.cuh"

#include <cfloat>

namespace rb200 {

namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_STAGES = 4;
constexpr int ATT_ROWS = kAttentionTileRows;       // query vectors per CTA: one m16 tile per warp

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attention_mma_kernel(const float * __restrict__ qkv, int ld, int n_head, KvLayout kv, int layer,
                                                                    const int2 * __restrict__ items, const int32_t * __restrict__ tok_slot,
                                                                    const int32_t * __restrict__ tok_pos, const int32_t * __restrict__ tok_pos_min,
                                                                    float * __restrict__ out, int ldo, int skip_small) {
    constexpr int PANELS = HD / 64;            // 128-byte panels per row
    constexpr int KSTEPS = HD / 16;
    constexpr int NT = HD / 8;
    constexpr int Q_BYTES = PANELS * ATT_ROWS * 128;
    constexpr int TILE_BYTES = PANELS * 16 * 128;          // one K or V block: 16 tokens x HD f16
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t * q_hi = smem;
    uint8_t * q_lo = smem + Q_BYTES;
    uint8_t * kv_s = smem + 2 * Q_BYTES;                    // [stage][K | V]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int hk = blockIdx.y;
    const int G = n_head / kv.n_head_kv;
    // items are listed in row order (decode rows first, long prefill chunks last): walk them backwards so
    // the longest-running CTAs start first and the one-token rows fill the tail
    const int2 item = items[gridDim.x - 1 - blockIdx.x];
    const int i0 = item.x, ntok = item.y;
    if (skip_small && ntok * G <= 16) return;       // served by the split-KV kernel below
    const int slot = tok_slot[i0], pos0 = tok_pos[i0], pmin = tok_pos_min[i0];
    const int last = pos0 + ntok - 1;
    const int32_t * table = kv.block_table + (size_t)slot * kv.max_blocks;
    const __half * kbase = kv.k + layer * kv.layer_stride;
    const __half * vbase = kv.v + layer * kv.layer_stride;
    const float scale = rsqrtf((float)HD);

    // ---- stage the query tile as hi + lo f16
    {
        const int R = tid >> 1, part = tid & 1;
        const int tt = R / G, hg = R % G;
        const bool valid = tt < ntok;
        const float * src = qkv + (size_t)(i0 + (valid ? tt : 0)) * ld + (size_t)(hk * G + hg) * HD + part * (HD / 2);
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) {          // chunks of 8 columns in this thread's half row
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
            const uint32_t off = (uint32_t)((col_chunk >> 3) * (ATT_ROWS * 128)) + swz(R, col_chunk & 7);
            *reinterpret_cast<uint4 *>(q_hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4 *>(q_lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
        }
    }

    const int nb0 = pmin >> 4, nb1 = last >> 4;
    const int n_blocks = nb1 - nb0 + 1;
    auto load_block = [&](int bi, int stage) {
        const int blk = rb_block(kv, table[nb0 + bi]);
        const size_t base = ((size_t)blk * kv.n_head_kv + hk) * 16 * HD;
        const uint32_t k_s = smem_u32(kv_s + stage * 2 * TILE_BYTES);
        const uint32_t v_s = k_s + TILE_BYTES;
#pragma unroll
        for (int i = 0; i < (16 * HD / 8 + ATT_THREADS - 1) / ATT_THREADS; ++i) {
            const int c = tid + i * ATT_THREADS;                 // 16-byte chunk of the tile
            if (c >= 16 * HD / 8) break;                         // fewer chunks than threads (head_dim 64)
            const int token = c / (HD / 8), dchunk = c % (HD / 8);
            const uint32_t off = (uint32_t)((dchunk >> 3) * (16 * 128)) + swz(token, dchunk & 7);
            cp_async16(k_s + off, kbase + base + (size_t)c * 8, 16);
            cp_async16(v_s + off, vbase + base + (size_t)c * 8, 16);
        }
    };
#pragma unroll
    for (int s = 0; s < ATT_STAGES - 1; ++s) {
        if (s < n_blocks) load_block(s, s);
        cp_async_commit();
    }
    __syncthreads();

    uint32_t qh[KSTEPS][4], ql[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        const uint32_t off = (uint32_t)((ks >> 2) * (ATT_ROWS * 128)) + swz(warp * 16 + (lane & 15), (ks & 3) * 2 + (lane >> 4));
        ldmatrix_x4(smem_u32(q_hi) + off, qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3]);
        ldmatrix_x4(smem_u32(q_lo) + off, ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3]);
    }

    const int R0 = warp * 16 + g, R1 = R0 + 8;
    const int tt0 = R0 / G, tt1 = R1 / G;
    const int prow0 = tt0 < ntok ? pos0 + tt0 : -1;      // last position this query row may see
    const int prow1 = tt1 < ntok ? pos0 + tt1 : -1;

    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int bi = 0; bi < n_blocks; ++bi) {
        cp_async_wait<ATT_STAGES - 2>();
        __syncthreads();
        const int nxt = bi + ATT_STAGES - 1;
        if (nxt < n_blocks) load_block(nxt, nxt % ATT_STAGES);
        cp_async_commit();

        const uint32_t k_s = smem_u32(kv_s + (bi % ATT_STAGES) * 2 * TILE_BYTES);
        const uint32_t v_s = k_s + TILE_BYTES;
        // four independent accumulator chains (two key octets x query hi / lo) instead of two twice as deep
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, sl[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t b0, b1, b2, b3;
            const uint32_t off = (uint32_t)((ks >> 2) * (16 * 128)) + swz((lane & 7) + ((lane >> 4) << 3), (ks & 3) * 2 + ((lane >> 3) & 1));
            ldmatrix_x4(k_s + off, b0, b1, b2, b3);
            mma_f16(s[0], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b0, b1);
            mma_f16(s[1], qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3], b2, b3);
            mma_f16(sl[0], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b0, b1);
            mma_f16(sl[1], ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3], b2, b3);
        }
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[ni][e] += sl[ni][e];
        // causal mask by position within the slot
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
        const float c0 = expf(m0 - ref0), c1 = expf(m1 - ref1);      // exp(-inf) = 0 for the first block
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
            pl[f] = pack_half2(x0 - back.x, x1 - back.y);
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
    if (tt0 < ntok) {
        const float inv = 1.0f / l0;
        float * dst = out + (size_t)(i0 + tt0) * ldo + (size_t)(hk * G + R0 % G) * HD + 2 * tq;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) *reinterpret_cast<float2 *>(dst + nt * 8) = make_float2(o[nt][0] * inv, o[nt][1] * inv);
    }
    if (tt1 < ntok) {
        const float inv = 1.0f / l1;
        float * dst = out + (size_t)(i0 + tt1) * ldo + (size_t)(hk * G + R1 % G) * HD + 2 * tq;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) *reinterpret_cast<float2 *>(dst + nt * 8) = make_float2(o[nt][2] * inv, o[nt][3] * inv);
    }
}

template <int HD>
void launch_hd(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items, const int32_t * tok_slot,
               const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int skip_small, cudaStream_t stream) {
    constexpr int smem = 2 * (HD / 64) * ATT_ROWS * 128 + ATT_STAGES * 2 * (HD / 64) * 16 * 128;
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(attention_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    attention_mma_kernel<HD><<<dim3(n_items, kv.n_head_kv), ATT_THREADS, smem, stream>>>(qkv, ld, n_head, kv, layer, items, tok_slot, tok_pos,
                                                                                       tok_pos_min, out, ldo, skip_small);
}

} // namespace

bool attention_mma_supported(int n_head, int n_head_kv, int head_dim, int block_tokens) {
    const int G = n_head / n_head_kv;
    return (head_dim == 64 || head_dim == 128) && block_tokens == 16 && n_head % n_head_kv == 0 && (G == 1 || G == 2 || G == 4 || G == 8 || G == 16);
}

void launch_attention_mma(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items, const int32_t * tok_slot,
                          const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, bool skip_small, cudaStream_t stream) {
    if (n_items <= 0) return;
    if (kv.head_dim == 128) launch_hd<128>(qkv, ld, n_head, kv, layer, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, skip_small, stream);
    else launch_hd<64>(qkv, ld, n_head, kv, layer, items, n_items, tok_slot, tok_pos, tok_pos_min, out, ldo, skip_small, stream);
}

} // namespace rb200
