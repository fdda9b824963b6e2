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
    if (configured.first()) {
        cudaFuncSetAttribute(attention_decode8_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
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
