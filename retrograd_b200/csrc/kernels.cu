// Reference-grade CUDA kernels of the decode step: packing maps, block-table resolution,
// embedding gather, RMSNorm, dequant-fused row GEMM, RoPE + paged KV store, paged attention,
// SwiGLU, MoE routing, per-row LoRA. These are the simple, shape-agnostic implementations every
// tuned kernel is checked against on the device; the tuned streaming kernels live in their own
// files and take over for the shapes they cover.

#include "kernels.cuh"
#include "blocks.hpp"
#include "split_emit.cuh"

#include <algorithm>
#include <cfloat>
#include <type_traits>

namespace rb200 {

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ __forceinline__ float e8m0_half_dev(uint8_t x) {
    const uint32_t bits = x == 0 ? 0x00200000u : x == 1 ? 0x00400000u : ((uint32_t)x - 1) << 23;
    return __uint_as_float(bits);
}

__constant__ float c_fp4_doubled[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};

// Decodes 8 consecutive elements starting at k (k % 8 == 0) of a stored row.
template <uint32_t TYPE>
__device__ __forceinline__ void decode8(const uint8_t * __restrict__ row, uint32_t k, float (&w)[8]) {
    if constexpr (TYPE == GGML_F32) {
        const float4 a = *reinterpret_cast<const float4 *>(row + (size_t)k * 4);
        const float4 b = *reinterpret_cast<const float4 *>(row + (size_t)k * 4 + 16);
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else if constexpr (TYPE == GGML_F16) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(row + (size_t)k * 2);
        const __half2 * h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            w[2 * i] = f.x;
            w[2 * i + 1] = f.y;
        }
    } else if constexpr (TYPE == GGML_BF16) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(row + (size_t)k * 2);
        const uint16_t * h = reinterpret_cast<const uint16_t *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = __uint_as_float((uint32_t)h[i] << 16);
    } else if constexpr (TYPE == GGML_Q8_0) {
        const uint8_t * b = row + (size_t)(k >> 5) * 34;
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        const uint8_t * q = b + 2 + (k & 31);
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = d * (float)(int8_t)q[i];
    } else if constexpr (TYPE == GGML_Q4_K) {
        const uint8_t * b = row + (size_t)(k >> 8) * 144;
        const uint32_t in = k & 255;
        const uint32_t grp = in >> 6, hi = (in >> 5) & 1, l = in & 31;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(b));
        const float dmin = half_bits_to_float(*reinterpret_cast<const uint16_t *>(b + 2));
        const uint8_t * s = b + 4;
        const int j = 2 * grp + hi;
        uint32_t sc, mn;
        if (j < 4) {
            sc = s[j] & 63;
            mn = s[j + 4] & 63;
        } else {
            sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
            mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
        }
        const float dl = d * (float)sc, ml = dmin * (float)mn;
        const uint8_t * q = b + 16 + grp * 32 + l;
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = dl * (float)((q[i] >> (4 * hi)) & 0xF) - ml;
    } else if constexpr (TYPE == GGML_MXFP4) {
        const uint8_t * b = row + (size_t)(k >> 5) * 17;
        const uint32_t in = k & 31, hi = in >> 4, l = in & 15;
        const float d = e8m0_half_dev(b[0]);
        const uint8_t * q = b + 1 + l;
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = d * c_fp4_doubled[(q[i] >> (4 * hi)) & 0xF];
    }
}

// ------------------------------------------------------------------------------------------
// Packing: step plan -> batch maps, with block tables resolved to physical KV cells.

__global__ void pack_scan_kernel(const RowDesc * __restrict__ rows, int n_rows, int tile_tokens, int32_t * __restrict__ cu,
                                 int32_t * __restrict__ out_rank, int32_t * __restrict__ tile_rank) {
    __shared__ int32_t warp_tok[32], warp_out[32], warp_tile[32];
    __shared__ int32_t carry_tok, carry_out, carry_tile;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid == 0) { carry_tok = 0; carry_out = 0; carry_tile = 0; }
    __syncthreads();
    for (int base = 0; base < n_rows; base += blockDim.x) {
        const int r = base + tid;
        const int32_t n = r < n_rows ? rows[r].n : 0;
        const int32_t s = r < n_rows ? (rows[r].sample != 0) : 0;
        const int32_t nt = (n + tile_tokens - 1) / tile_tokens;
        int32_t in = n, is = s, it = nt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t a = __shfl_up_sync(0xffffffffu, in, o);
            const int32_t b = __shfl_up_sync(0xffffffffu, is, o);
            const int32_t c = __shfl_up_sync(0xffffffffu, it, o);
            if (lane >= o) { in += a; is += b; it += c; }
        }
        if (lane == 31) { warp_tok[wid] = in; warp_out[wid] = is; warp_tile[wid] = it; }
        __syncthreads();
        if (wid == 0) {
            int32_t a = warp_tok[lane], b = warp_out[lane], c = warp_tile[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int32_t ua = __shfl_up_sync(0xffffffffu, a, o);
                const int32_t ub = __shfl_up_sync(0xffffffffu, b, o);
                const int32_t uc = __shfl_up_sync(0xffffffffu, c, o);
                if (lane >= o) { a += ua; b += ub; c += uc; }
            }
            warp_tok[lane] = a;
            warp_out[lane] = b;
            warp_tile[lane] = c;
        }
        __syncthreads();
        const int32_t pre_tok = carry_tok + (wid ? warp_tok[wid - 1] : 0);
        const int32_t pre_out = carry_out + (wid ? warp_out[wid - 1] : 0);
        const int32_t pre_tile = carry_tile + (wid ? warp_tile[wid - 1] : 0);
        if (r < n_rows) {
            cu[r] = pre_tok + in - n;
            out_rank[r] = pre_out + is - s;
            tile_rank[r] = pre_tile + it - nt;
        }
        __syncthreads();
        if (tid == 0) {
            carry_tok += warp_tok[31];
            carry_out += warp_out[31];
            carry_tile += warp_tile[31];
        }
        __syncthreads();
    }
    if (tid == 0) {
        cu[n_rows] = carry_tok;
        out_rank[n_rows] = carry_out;
        tile_rank[n_rows] = carry_tile;
    }
}

__global__ void pack_fill_kernel(const RowDesc * __restrict__ rows, int n_rows, int n_tokens, const int32_t * __restrict__ block_table,
                                 int max_blocks, int block_tokens, int tile_tokens, PackMaps maps) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens) return;
    int lo = 0, hi = n_rows - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (maps.cu_rows[mid] <= i) lo = mid; else hi = mid - 1;
    }
    const RowDesc row = rows[lo];
    const int j = i - maps.cu_rows[lo];
    const int pos = row.pos0 + j;
    RB_CHECK(maps.check, CHECK_SLOT, row.slot, maps.n_slots, return);
    RB_CHECK(maps.check, CHECK_ADAPTER, row.adapter + 1, maps.n_adapters + 1, return);      // -1 = none
    RB_CHECK(maps.check, CHECK_POSITION, pos, (long long)max_blocks * block_tokens, return);
    maps.tok_slot[i] = row.slot;
    maps.tok_pos[i] = pos;
    maps.tok_row[i] = lo;
    maps.tok_adapter[i] = row.adapter;
    maps.tok_pos_min[i] = row.pos_min;
    const int blk = block_table[(size_t)row.slot * max_blocks + pos / block_tokens];
    RB_CHECK(maps.check, CHECK_BLOCK, blk, maps.n_blocks, return);
    maps.tok_cell[i] = blk * block_tokens + pos % block_tokens;
    if (row.sample && j == row.n - 1) maps.out_index[maps.out_rank[lo]] = i;
    if (j % tile_tokens == 0) maps.attn_items[maps.tile_rank[lo] + j / tile_tokens] = make_int2(i, min(tile_tokens, row.n - j));
}

__global__ void block_table_patch_kernel(int32_t * __restrict__ table, const int32_t * __restrict__ patches, int n, int table_entries, int n_blocks,
                                         int * check) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    RB_CHECK(check, CHECK_TABLE_INDEX, patches[2 * i], table_entries, return);
    RB_CHECK(check, CHECK_BLOCK, patches[2 * i + 1], n_blocks, return);
    table[patches[2 * i]] = patches[2 * i + 1];
}

// Copies whole KV blocks (all layers, K and V) for copy-on-write of a shared boundary block.
__global__ void kv_block_copy_kernel(KvLayout kv, int n_layer, const int32_t * __restrict__ pairs) {
    const int pair = blockIdx.x, layer = blockIdx.y;
    const int32_t src = pairs[2 * pair], dst = pairs[2 * pair + 1];
    RB_CHECK(kv.check, CHECK_BLOCK, src, kv.n_blocks, return);
    RB_CHECK(kv.check, CHECK_BLOCK, dst, kv.n_blocks, return);
    const bool quant = kv.storage != KV_F16;
    // bytes of one block (rows are multiples of 8 bytes, a block holds block_tokens = 16 of them per head)
    const size_t block_bytes = (size_t)kv.n_head_kv * kv.block_tokens * (quant ? (size_t)kv.q_row_bytes : (size_t)kv.head_dim * 2);
    const uint8_t * kbase = quant ? kv.kq + layer * kv.q_layer_stride : reinterpret_cast<const uint8_t *>(kv.k + layer * kv.layer_stride);
    const uint8_t * vbase = quant ? kv.vq + layer * kv.q_layer_stride : reinterpret_cast<const uint8_t *>(kv.v + layer * kv.layer_stride);
    const uint2 * ks = reinterpret_cast<const uint2 *>(kbase + src * block_bytes);
    uint2 * kd = reinterpret_cast<uint2 *>(const_cast<uint8_t *>(kbase) + dst * block_bytes);
    const uint2 * vs = reinterpret_cast<const uint2 *>(vbase + src * block_bytes);
    uint2 * vd = reinterpret_cast<uint2 *>(const_cast<uint8_t *>(vbase) + dst * block_bytes);
    const size_t n8 = block_bytes / 8;
    for (size_t i = threadIdx.x; i < n8; i += blockDim.x) {
        kd[i] = ks[i];
        vd[i] = vs[i];
    }
    (void)n_layer;
}

// Moves the cells of one slot between the paged cache and a dense [layer][K|V][pos][head][row]
// buffer (sequence snapshots); a row is head_dim f16 values or the quantised pool's row bytes. grid = (positions, layers * 2).
__global__ void kv_snapshot_kernel(KvLayout kv, const int32_t * __restrict__ table, int pos_first, uint16_t * __restrict__ dense, int n_pos,
                                   int to_cache) {
    const int p = blockIdx.x, layer = blockIdx.y >> 1, is_v = blockIdx.y & 1;
    const int pos = pos_first + p;
    RB_CHECK(kv.check, CHECK_POSITION, pos, (long long)kv.max_blocks * kv.block_tokens, return);
    const int blk = table[pos / kv.block_tokens], off = pos % kv.block_tokens;
    RB_CHECK(kv.check, CHECK_BLOCK, blk, kv.n_blocks, return);
    const bool quant = kv.storage != KV_F16;
    const int row_u16 = quant ? kv.q_row_bytes / 2 : kv.head_dim;         // 16-bit words per (cell, head) row
    uint16_t * cache = quant ? reinterpret_cast<uint16_t *>((is_v ? kv.vq : kv.kq) + layer * kv.q_layer_stride)
                             : reinterpret_cast<uint16_t *>((is_v ? kv.v : kv.k) + layer * kv.layer_stride);
    const int row = kv.n_head_kv * row_u16;
    uint16_t * d = dense + ((size_t)blockIdx.y * n_pos + p) * row;
    for (int idx = threadIdx.x; idx < row; idx += blockDim.x) {
        const int h = idx / row_u16, i = idx % row_u16;
        const size_t c = (((size_t)blk * kv.n_head_kv + h) * kv.block_tokens + off) * row_u16 + i;
        if (to_cache) cache[c] = d[idx]; else d[idx] = cache[c];
    }
}

// Quantised KV pools: the step's K rows (after RoPE) and V rows from the qkv buffer into the pool. One CTA per token,
// a warp per 32-element block of a head row in turn, lane j its element j: the arithmetic of ggml's reference
// quantisers (quantize_row_q8_0_ref: d = amax / 127, q = roundf(x / d); quantize_row_q4_0_ref: d = the element of
// largest magnitude (the first of equals) / -8, q = min(15, (int)(x / d + 8.5))), the scale stored as f16.
__global__ void kv_quant_store_kernel(const float * __restrict__ qkv, int ld, int n_head, KvLayout kv, int layer, const int32_t * __restrict__ tok_cell) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, per_head = kv.head_dim / 32;
    const int cell = tok_cell[t];
    RB_CHECK(kv.check, CHECK_CELL, cell, (long long)kv.n_blocks * kv.block_tokens, return);
    const int blk = cell / kv.block_tokens, off = cell % kv.block_tokens;
    // the token's K heads, then its V heads, are one run of 2 * n_head_kv * head_dim values behind its q heads; a warp
    // takes four of the run's 32-value blocks per pass, their loads issued together
    const int n_qb = 2 * kv.n_head_kv * per_head, n_warps = blockDim.x >> 5;
    const float * run = qkv + (size_t)t * ld + (size_t)n_head * kv.head_dim;
    for (int qb0 = threadIdx.x >> 5; qb0 < n_qb; qb0 += 4 * n_warps) {
    float xs[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) xs[u] = qb0 + u * n_warps < n_qb ? run[(size_t)(qb0 + u * n_warps) * 32 + lane] : 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
    const int qb = qb0 + u * n_warps;
    if (qb >= n_qb) break;
    const int hh = qb / per_head, b = qb % per_head;                    // quant block b of head row hh (K heads, then V heads)
    const int is_v = hh >= kv.n_head_kv ? 1 : 0, h = hh - is_v * kv.n_head_kv;
    const float x = xs[u];
    uint8_t * row = (is_v ? kv.vq : kv.kq) + layer * kv.q_layer_stride + (((size_t)blk * kv.n_head_kv + h) * kv.block_tokens + off) * kv.q_row_bytes;
    float a = fabsf(x);
    int who = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, o);
        const int ow = __shfl_xor_sync(0xffffffffu, who, o);
        if (oa > a || (oa == a && ow < who)) { a = oa; who = ow; }
    }
    if (kv.storage == KV_Q8_0) {
        const float d = a / 127.f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        row[b * 32 + lane] = (uint8_t)(int8_t)(int)roundf(x * id);
        if (lane == 0) reinterpret_cast<__half *>(row + kv.head_dim)[b] = __float2half_rn(d);
    } else {
        const float mx = __shfl_sync(0xffffffffu, x, who);
        const float d = mx / -8.f;
        const float id = d != 0.f ? 1.0f / d : 0.f;
        const int q = min(15, (int)(int8_t)(x * id + 8.5f));
        const int hi = __shfl_down_sync(0xffffffffu, q, 16);
        if (lane < 16) row[b * 16 + lane] = (uint8_t)(q | (hi << 4));
        if (lane == 0) reinterpret_cast<__half *>(row + kv.head_dim / 2)[b] = __float2half_rn(d);
    }
    }
    }
}

// Quantised KV pools: every pool block row r of the step may attend to, dequantised (scale * quant in f32, rounded
// to f16) into the one-layer f16 scratch under the same block number. grid (rows that need it, unit strides).
__global__ void kv_dequant_kernel(KvLayout kv, int layer, int n_rows, const int32_t * __restrict__ cu_rows, const int32_t * __restrict__ tok_slot,
                                  const int32_t * __restrict__ tok_pos, const int32_t * __restrict__ tok_pos_min, int skip_tokens) {
    // blockIdx.x counts the rows of more than skip_tokens tokens (shorter rows are read from the pool by a kernel that
    // decodes it itself): find that row - every warp the same way, 32 rows per ballot
    int row = -1;
    {
        const int lane = threadIdx.x & 31;
        int seen = 0;
        for (int r0 = 0; r0 < n_rows && row < 0; r0 += 32) {
            const int r = r0 + lane;
            const bool needy = r < n_rows && cu_rows[r + 1] - cu_rows[r] > skip_tokens;
            const unsigned mask = __ballot_sync(0xffffffffu, needy);
            const int here = __popc(mask);
            if (seen + here > (int)blockIdx.x) {
                unsigned m = mask;
                for (int k = (int)blockIdx.x - seen; k > 0; --k) m &= m - 1;        // drop the k lowest set bits
                row = r0 + __ffs(m) - 1;
            }
            seen += here;
        }
    }
    if (row < 0) return;
    const int i0 = cu_rows[row], n = cu_rows[row + 1] - i0;
    const int slot = tok_slot[i0], last = tok_pos[i0] + n - 1, pmin = tok_pos_min[i0];
    const int hd = kv.head_dim, rows = kv.n_head_kv * kv.block_tokens;          // (head, cell) rows of the block
    const bool q8 = kv.storage == KV_Q8_0;
    const int words = q8 ? hd / 4 : hd / 8;                                      // 32-bit words of quants per row
    // a unit of work: the 16 cells of one head of K or V of one block; the row's CTAs take units in strides of grid.y
    const int b_first = pmin / kv.block_tokens, n_units = (last / kv.block_tokens - b_first + 1) * 2 * kv.n_head_kv;
    for (int unit = blockIdx.y; unit < n_units; unit += gridDim.y) {
    const int bi = b_first + unit / (2 * kv.n_head_kv), is_v = (unit / kv.n_head_kv) & 1, h = unit % kv.n_head_kv;
    const int blk = rb_block(kv, kv.block_table[(size_t)slot * kv.max_blocks + bi]);
    for (int idx = threadIdx.x; idx < kv.block_tokens * words; idx += blockDim.x) {
        const int w = idx % words, r = h * kv.block_tokens + idx / words;
        const uint8_t * row = (is_v ? kv.vq : kv.kq) + layer * kv.q_layer_stride + ((size_t)blk * rows + r) * kv.q_row_bytes;
        __half * dst = (is_v ? kv.v : kv.k) + ((size_t)blk * rows + r) * hd;
        const uint32_t word = reinterpret_cast<const uint32_t *>(row)[w];
        if (q8) {
            const float d = __half2float(reinterpret_cast<const __half *>(row + hd)[w / 8]);
            __half2 o[2];
            o[0] = __floats2half2_rn(d * (float)(int8_t)(word & 0xff), d * (float)(int8_t)((word >> 8) & 0xff));
            o[1] = __floats2half2_rn(d * (float)(int8_t)((word >> 16) & 0xff), d * (float)(int8_t)(word >> 24));
            *reinterpret_cast<uint2 *>(dst + 4 * w) = *reinterpret_cast<const uint2 *>(o);
        } else {
            // word w: bytes 4 (w % 4) .. + 3 of block w / 4; a byte's low nibble is element j, its high nibble element j + 16
            const int b = w / 4, j = 4 * (w % 4);
            const float d = __half2float(reinterpret_cast<const __half *>(row + hd / 2)[b]);
            __half2 lo[2], hi[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t b0 = (word >> (16 * e)) & 0xff, b1 = (word >> (16 * e + 8)) & 0xff;
                lo[e] = __floats2half2_rn(d * (float)((int)(b0 & 15) - 8), d * (float)((int)(b1 & 15) - 8));
                hi[e] = __floats2half2_rn(d * (float)((int)(b0 >> 4) - 8), d * (float)((int)(b1 >> 4) - 8));
            }
            *reinterpret_cast<uint2 *>(dst + b * 32 + j) = *reinterpret_cast<const uint2 *>(lo);
            *reinterpret_cast<uint2 *>(dst + b * 32 + 16 + j) = *reinterpret_cast<const uint2 *>(hi);
        }
    }
    }
}

// ------------------------------------------------------------------------------------------

template <uint32_t TYPE>
__global__ void embed_kernel(WeightView e, const int32_t * __restrict__ tokens, float * __restrict__ x, int * check) {
    const int t = blockIdx.x;
    RB_CHECK(check, CHECK_TOKEN, tokens[t], e.n_out, return);
    const uint8_t * row = e.data + (size_t)tokens[t] * e.row_bytes;
    for (uint32_t k = threadIdx.x * 8; k < e.n_in; k += blockDim.x * 8) {
        float w[8];
        decode8<TYPE>(row, k, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[(size_t)t * e.n_in + k + i] = w[i];
    }
}

__global__ void rms_norm_kernel(const float * __restrict__ x, int ldx, const int32_t * __restrict__ gather, const float * __restrict__ w, int n,
                                float eps, float * __restrict__ y, int ldy, SplitAct split) {
    pdl_trigger();      // the next kernel's prologue (weight prefetch) may overlap this kernel
    pdl_wait();
    __shared__ float partial[32];
    const int t = blockIdx.x;
    const float * xr = x + (size_t)(gather ? gather[t] : t) * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) partial[0] = v;
    }
    __syncthreads();
    const float scale = 1.0f / sqrtf(partial[0] / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i] * scale * w[i];
        if (y) y[(size_t)t * ldy + i] = v;
        if (split.hi) emit_split(split, t, i, v);
    }
}

// The same with four columns per thread (n % 32 == 0, rows 16-byte aligned); y may be null when only
// the split form is consumed.
__global__ void rms_norm4_kernel(const float * __restrict__ x, int ldx, const int32_t * __restrict__ gather, const float * __restrict__ w, int n,
                                 float eps, float * __restrict__ y, int ldy, SplitAct split) {
    pdl_trigger();      // the next kernel's prologue (weight prefetch) may overlap this kernel
    pdl_wait();
    __shared__ float partial[32];
    const int t = blockIdx.x;
    const float * xr = x + (size_t)(gather ? gather[t] : t) * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) partial[0] = v;
    }
    __syncthreads();
    const float scale = 1.0f / sqrtf(partial[0] / (float)n + eps);
    for (int base = 0; base < n; base += blockDim.x * 4) {
        const int i = base + threadIdx.x * 4;
        const bool active = i < n;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (active) {
            const float4 a = *reinterpret_cast<const float4 *>(xr + i), b = *reinterpret_cast<const float4 *>(w + i);
            v = make_float4(a.x * scale * b.x, a.y * scale * b.y, a.z * scale * b.z, a.w * scale * b.w);
            if (y) *reinterpret_cast<float4 *>(y + (size_t)t * ldy + i) = v;
        }
        if (split.hi) emit_split4(split, t, i, v, active);
    }
}

// One warp per output row and group of eight tokens: grid (token groups, row blocks) - the token group is
// the fastest grid dimension, so the CTAs that decode the same rows run together and share them in L2.
template <uint32_t TYPE>
__global__ void gemm_rows_kernel(WeightView w, const float * __restrict__ x, int ldx, int n_tokens, float * __restrict__ y, int ldy,
                                 const float * __restrict__ bias, const float * __restrict__ residual, int ldr) {
    const int lane = threadIdx.x & 31;
    const uint32_t o = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (o >= w.n_out) return;
    const uint8_t * row = w.data + (size_t)o * w.row_bytes;
    for (int t0 = blockIdx.x * 8; t0 < n_tokens; t0 += gridDim.x * 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (uint32_t k = lane * 8; k < w.n_in; k += 256) {
            float wv[8];
            decode8<TYPE>(row, k, wv);
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                if (t0 + tt < n_tokens) {
                    const float4 a = *reinterpret_cast<const float4 *>(x + (size_t)(t0 + tt) * ldx + k);
                    const float4 b = *reinterpret_cast<const float4 *>(x + (size_t)(t0 + tt) * ldx + k + 4);
                    acc[tt] += wv[0] * a.x + wv[1] * a.y + wv[2] * a.z + wv[3] * a.w + wv[4] * b.x + wv[5] * b.y + wv[6] * b.z + wv[7] * b.w;
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < 8; ++tt) {
            const float v = warp_sum(acc[tt]);
            if (lane == 0 && t0 + tt < n_tokens) {
                float r = v;
                if (bias) r += bias[o];
                if (residual) r += residual[(size_t)(t0 + tt) * ldr + o];
                y[(size_t)(t0 + tt) * ldy + o] = r;
            }
        }
    }
}

// qkv row layout: [q: n_head*hd | k: n_head_kv*hd | v: n_head_kv*hd]. Grid (tokens, groups of eight
// rotated heads): a block rotates its heads in place, then stores the K heads among them into the
// cache; the blocks of group 0 also store the token's V heads.
__global__ void rope_store_kernel(float * __restrict__ qkv, int ld, int n_head, int n_head_kv, int head_dim, int n_rot, int neox,
                                  const float * __restrict__ inv_freq, const int32_t * __restrict__ tok_pos, const int32_t * __restrict__ tok_cell,
                                  KvLayout kv, int layer, const float * __restrict__ partial, int n_chunks, int t_stride, int ld_partial,
                                  const float * __restrict__ bias) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    float * row = qkv + (size_t)t * ld;
    const int pos = tok_pos[t];
    const int half_rot = n_rot / 2;
    const int n_rot_heads = n_head + n_head_kv;
    const int h_lo = blockIdx.y * 8, h_hi = min(n_rot_heads, h_lo + 8);
    if (partial) {
        // the block's columns of the row (its heads; block 0 also the V heads) from the GEMM's partial
        // sums, four columns per thread, every chunk's load issued before the first addition
        const size_t chunk_stride = (size_t)t_stride * ld_partial;
        const int v_lo = n_rot_heads * head_dim, v_hi = v_lo + n_head_kv * head_dim;
        for (int part = 0; part < (blockIdx.y == 0 ? 2 : 1); ++part) {
            const int c_lo = part ? v_lo : h_lo * head_dim, c_hi = part ? v_hi : h_hi * head_dim;
            for (int col = c_lo + threadIdx.x * 4; col < c_hi; col += blockDim.x * 4) {
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c0 = 0; c0 < n_chunks; c0 += 8) {
                    float4 p[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        p[c] = c0 + c < n_chunks ? *reinterpret_cast<const float4 *>(partial + (size_t)(c0 + c) * chunk_stride + (size_t)t * ld_partial + col)
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        if (c0 + c < n_chunks) { sum.x += p[c].x; sum.y += p[c].y; sum.z += p[c].z; sum.w += p[c].w; }
                    }
                }
                if (bias) {
                    const float4 b = *reinterpret_cast<const float4 *>(bias + col);
                    sum.x += b.x; sum.y += b.y; sum.z += b.z; sum.w += b.w;
                }
                *reinterpret_cast<float4 *>(row + col) = sum;
            }
        }
        __syncthreads();
    }
    for (int idx = threadIdx.x; idx < (h_hi - h_lo) * half_rot; idx += blockDim.x) {
        const int h = h_lo + idx / half_rot, i = idx % half_rot;
        float * p = row + (size_t)h * head_dim;   // k heads follow the q heads contiguously
        const float theta = (float)pos * inv_freq[i];
        float s, c;
        sincosf(theta, &s, &c);
        const int i0 = neox ? i : 2 * i, i1 = neox ? i + half_rot : 2 * i + 1;
        const float a = p[i0], b = p[i1];
        p[i0] = a * c - b * s;
        p[i1] = a * s + b * c;
    }
    __syncthreads();
    const int cell = tok_cell[t];
    RB_CHECK(kv.check, CHECK_CELL, cell, (long long)kv.n_blocks * kv.block_tokens, return);
    const int blk = cell / kv.block_tokens, off = cell % kv.block_tokens;
    const float * ksrc = row + (size_t)n_head * head_dim;
    const float * vsrc = ksrc + (size_t)n_head_kv * head_dim;
    __half * kdst = kv.k + layer * kv.layer_stride;
    __half * vdst = kv.v + layer * kv.layer_stride;
    const int k_lo = max(h_lo, n_head) - n_head, k_hi = h_hi - n_head;       // K heads rotated by this block
    for (int idx = threadIdx.x + k_lo * head_dim; idx < k_hi * head_dim; idx += blockDim.x) {
        const int h = idx / head_dim, i = idx % head_dim;
        kdst[(((size_t)blk * n_head_kv + h) * kv.block_tokens + off) * head_dim + i] = __float2half_rn(ksrc[idx]);
    }
    if (blockIdx.y == 0) {
        for (int idx = threadIdx.x; idx < n_head_kv * head_dim; idx += blockDim.x) {
            const int h = idx / head_dim, i = idx % head_dim;
            vdst[(((size_t)blk * n_head_kv + h) * kv.block_tokens + off) * head_dim + i] = __float2half_rn(vsrc[idx]);
        }
    }
}

// One warp per (token, q head); lanes own head dimensions; positions in groups of four.
__global__ void attention_ref_kernel(const float * __restrict__ qkv, int ld, int n_head, KvLayout kv, int layer,
                                     const int32_t * __restrict__ tok_slot, const int32_t * __restrict__ tok_pos,
                                     const int32_t * __restrict__ tok_pos_min, float * __restrict__ out, int ldo, SplitAct split) {
    const int lane = threadIdx.x & 31;
    const int h = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int t = blockIdx.y;
    if (h >= n_head) return;
    const int hd = kv.head_dim, B = kv.block_tokens;
    const int hk = h / (n_head / kv.n_head_kv);
    const int slot = tok_slot[t], p_last = tok_pos[t], p_first = tok_pos_min[t];
    const int32_t * table = kv.block_table + (size_t)slot * kv.max_blocks;
    const __half * kbase = kv.k + layer * kv.layer_stride;
    const __half * vbase = kv.v + layer * kv.layer_stride;
    constexpr int MAXD = 8;  // head_dim <= 256
    float q[MAXD], acc[MAXD];
    const float scale = rsqrtf((float)hd);
#pragma unroll
    for (int j = 0; j < MAXD; ++j) {
        const int i = lane + 32 * j;
        q[j] = i < hd ? qkv[(size_t)t * ld + (size_t)h * hd + i] * scale : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int p0 = p_first; p0 <= p_last; p0 += 4) {
        float s[4];
        const __half * vp[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int p = p0 + u;
            s[u] = 0.f;
            vp[u] = nullptr;
            if (p <= p_last) {
                const int blk = rb_block(kv, table[p / B]);
                const size_t base = (((size_t)blk * kv.n_head_kv + hk) * B + p % B) * hd;
                const __half * kp = kbase + base;
                vp[u] = vbase + base;
#pragma unroll
                for (int j = 0; j < MAXD; ++j) {
                    const int i = lane + 32 * j;
                    if (i < hd) s[u] += q[j] * __half2float(kp[i]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) s[u] = warp_sum(s[u]);
        float mn = m;
#pragma unroll
        for (int u = 0; u < 4; ++u) if (p0 + u <= p_last) mn = fmaxf(mn, s[u]);
        const float corr = expf(m - mn);
        l *= corr;
#pragma unroll
        for (int j = 0; j < MAXD; ++j) acc[j] *= corr;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (p0 + u <= p_last) {
                const float pr = expf(s[u] - mn);
                l += pr;
#pragma unroll
                for (int j = 0; j < MAXD; ++j) {
                    const int i = lane + 32 * j;
                    if (i < hd) acc[j] += pr * __half2float(vp[u][i]);
                }
            }
        }
        m = mn;
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int j = 0; j < MAXD; ++j) {
        const int i = lane + 32 * j;
        if (i < hd) out[(size_t)t * ldo + (size_t)h * hd + i] = acc[j] * inv;
        if (split.hi && 32 * j < hd) emit_split(split, t, h * hd + i, acc[j] * inv);
    }
}

// x [t][ld] f32 -> its SplitAct (n a multiple of 32)
// Row t of the split form is row gather[t] / gather_div of x (or row t without a gather list).
__global__ void split_prep_kernel(const float * __restrict__ x, int ldx, int n, SplitAct split, const int32_t * __restrict__ gather, int gather_div) {
    pdl_trigger();      // the next kernel's prologue (weight prefetch) may overlap this kernel
    pdl_wait();
    const int t = blockIdx.y;
    const int src = gather ? gather[t] / gather_div : t;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    emit_split(split, t, i, x[(size_t)src * ldx + i]);
}

__global__ void swiglu_kernel(const float * __restrict__ gu, int ld, int ff, float * __restrict__ h, int ldh, SplitAct split) {
    pdl_trigger();      // the next kernel's prologue (weight prefetch) may overlap this kernel
    pdl_wait();
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ff) return;
    const float g = gu[(size_t)t * ld + i], u = gu[(size_t)t * ld + ff + i];
    const float v = g / (1.0f + expf(-g)) * u;
    if (h) h[(size_t)t * ldh + i] = v;
    if (split.hi) emit_split(split, t, i, v);
}

__global__ void swiglu4_kernel(const float * __restrict__ gu, int ld, int ff, float * __restrict__ h, int ldh, SplitAct split) {
    pdl_trigger();      // the next kernel's prologue (weight prefetch) may overlap this kernel
    pdl_wait();
    const int t = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const bool active = i < ff;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
        const float4 g = *reinterpret_cast<const float4 *>(gu + (size_t)t * ld + i), u = *reinterpret_cast<const float4 *>(gu + (size_t)t * ld + ff + i);
        v = make_float4(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y, g.z / (1.0f + expf(-g.z)) * u.z,
                        g.w / (1.0f + expf(-g.w)) * u.w);
        if (h) *reinterpret_cast<float4 *>(h + (size_t)t * ldh + i) = v;
    }
    if (split.hi) emit_split4(split, t, i, v, active);
}

__global__ void split_prep4_kernel(const float * __restrict__ x, int ldx, int n, SplitAct split, const int32_t * __restrict__ gather, int gather_div) {
    pdl_trigger();      // the next kernel's prologue (weight prefetch) may overlap this kernel
    pdl_wait();
    const int t = blockIdx.y;
    const int src = gather ? gather[t] / gather_div : t;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const bool active = i < n;
    const float4 v = active ? *reinterpret_cast<const float4 *>(x + (size_t)src * ldx + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    emit_split4(split, t, i, v, active);
}

// ------------------------------------------------------------------------------------------
// MoE

// One warp per token: softmax over experts, then k picks by (probability desc, id asc).
__global__ void moe_route_kernel(const float * __restrict__ logits, int n_expert, int k, int n_tokens, int32_t * __restrict__ ids,
                                 float * __restrict__ weights) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    constexpr int MAXE = 8;  // up to 256 experts
    float p[MAXE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < MAXE; ++j) {
        const int e = lane + 32 * j;
        p[j] = e < n_expert ? logits[(size_t)t * n_expert + e] : -INFINITY;
        mx = fmaxf(mx, p[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAXE; ++j) {
        const int e = lane + 32 * j;
        p[j] = e < n_expert ? expf(p[j] - mx) : 0.f;
    }
    // serial-order sum over experts so the value matches a scalar loop
    for (int e = 0; e < n_expert; ++e) {
        const float v = __shfl_sync(0xffffffffu, p[e >> 5], e & 31);
        sum += v;
    }
#pragma unroll
    for (int j = 0; j < MAXE; ++j) p[j] = p[j] / sum;
    for (int pick = 0; pick < k; ++pick) {
        float best = -1.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < MAXE; ++j) {
            const int e = lane + 32 * j;
            if (e < n_expert && (p[j] > best || (p[j] == best && e < best_e))) { best = p[j]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (lane == 0) {
            ids[(size_t)t * k + pick] = best_e;
            weights[(size_t)t * k + pick] = best;
        }
        if ((best_e & 31) == lane) p[best_e >> 5] = -2.f;
    }
}

// The (token, expert) pairs of every expert, in pair order: offsets[n_expert + 1] and sorted[n_pairs].
// One block of 32 warps. The pair list is staged in shared memory 8192 pairs at a time; warp w owns experts
// w, w + 32, ... and walks the staged pairs 32 at a time: a ballot marks the lanes that hold one of its expert's
// pairs, and a lane's place among them is a population count, so the order inside an expert stays the pair order.
// Two such walks (count, then place) with a scan over the experts in between; n_expert <= 1024.
constexpr int kGroupChunk = 8192;
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t * __restrict__ pair_expert, int n_pairs, int n_expert,
                                                         int32_t * __restrict__ offsets, int32_t * __restrict__ sorted) {
    __shared__ int32_t s_off[1025];
    __shared__ int32_t s_pairs[kGroupChunk];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned below = (1u << lane) - 1u;
    for (int i = threadIdx.x; i <= n_expert; i += blockDim.x) s_off[i] = 0;
    for (int c0 = 0; c0 < n_pairs; c0 += kGroupChunk) {
        const int n = min(kGroupChunk, n_pairs - c0);
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) s_pairs[i] = pair_expert[c0 + i];
        __syncthreads();
        for (int e = warp; e < n_expert; e += 32) {
            int count = 0;
            for (int p0 = 0; p0 < n; p0 += 32) count += __popc(__ballot_sync(0xffffffffu, p0 + lane < n && s_pairs[p0 + lane] == e));
            if (lane == 0) s_off[e + 1] += count;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int i = 0; i < n_expert; ++i) s_off[i + 1] += s_off[i];
    __syncthreads();
    for (int i = threadIdx.x; i <= n_expert; i += blockDim.x) offsets[i] = s_off[i];
    // s_off[e] now walks forward as expert e's pairs are placed (its owner warp is the only writer)
    for (int c0 = 0; c0 < n_pairs; c0 += kGroupChunk) {
        const int n = min(kGroupChunk, n_pairs - c0);
        __syncthreads();
        if (n_pairs > kGroupChunk || c0 > 0)        // a single chunk is still staged from the counting walk
            for (int i = threadIdx.x; i < n; i += blockDim.x) s_pairs[i] = pair_expert[c0 + i];
        __syncthreads();
        for (int e = warp; e < n_expert; e += 32) {
            int at = s_off[e];
            for (int p0 = 0; p0 < n; p0 += 32) {
                const bool mine = p0 + lane < n && s_pairs[p0 + lane] == e;
                const unsigned hits = __ballot_sync(0xffffffffu, mine);
                if (mine) sorted[at + __popc(hits & below)] = c0 + p0 + lane;
                at += __popc(hits);
            }
            __syncwarp();
            if (lane == 0) s_off[e] = at;
        }
    }
}

// Grouped expert GEMM: grid (output row groups, experts). One warp per output row of ITS expert; the row
// is decoded once per eight of the expert's pairs: y[pair][o] = deq(W[expert])[o] . x[pair / x_div].
// Every (pair, row) dot product keeps the lane-strided accumulation order of a single-pair pass.
template <uint32_t TYPE>
__global__ void moe_gemm_grouped_kernel(WeightView w, uint64_t expert_stride, const int32_t * __restrict__ offsets,
                                        const int32_t * __restrict__ sorted, const float * __restrict__ x, int ldx, int x_div,
                                        float * __restrict__ y, int ldy) {
    const int lane = threadIdx.x & 31;
    const uint32_t o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int e = blockIdx.y;
    const int begin = offsets[e], end = offsets[e + 1];
    if (o >= w.n_out || begin == end) return;
    const uint8_t * row = w.data + (size_t)e * expert_stride + (size_t)o * w.row_bytes;
    for (int p0 = begin; p0 < end; p0 += 8) {
        int pair[8];
        const float * xr[8];
        float acc[8];
#pragma unroll
        for (int tt = 0; tt < 8; ++tt) {
            pair[tt] = p0 + tt < end ? sorted[p0 + tt] : -1;
            xr[tt] = x + (size_t)((pair[tt] < 0 ? 0 : pair[tt]) / x_div) * ldx;
            acc[tt] = 0.f;
        }
        for (uint32_t k = lane * 8; k < w.n_in; k += 256) {
            float wv[8];
            decode8<TYPE>(row, k, wv);
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                if (pair[tt] >= 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[tt] += wv[i] * xr[tt][k + i];
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < 8; ++tt) {
            const float v = warp_sum(acc[tt]);
            if (lane == 0 && pair[tt] >= 0) y[(size_t)pair[tt] * ldy + o] = v;
        }
    }
}

// out[t] = residual[t] + sum over the token's experts in ascending expert id of weight * y
__global__ void moe_combine_kernel(const float * __restrict__ y, int ld, const int32_t * __restrict__ ids, const float * __restrict__ weights,
                                   int k, int d, const float * __restrict__ residual, float * __restrict__ out) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d) return;
    float acc = 0.f;
    int prev = -1;
    for (int pick = 0; pick < k; ++pick) {
        int best = 0x7fffffff, best_j = 0;
        for (int j = 0; j < k; ++j) {
            const int e = ids[(size_t)t * k + j];
            if (e > prev && e < best) { best = e; best_j = j; }
        }
        prev = best;
        acc += weights[(size_t)t * k + best_j] * y[((size_t)t * k + best_j) * ld + i];
    }
    out[(size_t)t * d + i] = (residual ? residual[(size_t)t * d + i] : 0.f) + acc;
}

// ------------------------------------------------------------------------------------------
// Per-row LoRA

__global__ void lora_shrink_kernel(const float * __restrict__ a_stack, int r_max, int n_in, const int32_t * __restrict__ tok_adapter,
                                   const float * __restrict__ x, int ldx, float * __restrict__ tmp) {
    const int lane = threadIdx.x & 31;
    const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int t = blockIdx.y;
    if (j >= r_max) return;
    const int a = tok_adapter[t];
    float acc = 0.f;
    if (a >= 0) {
        const float * ar = a_stack + ((size_t)a * r_max + j) * n_in;
        for (int i = lane; i < n_in; i += 32) acc += ar[i] * x[(size_t)t * ldx + i];
    }
    acc = warp_sum(acc);
    if (lane == 0) tmp[(size_t)t * r_max + j] = acc;
}

// Segmented shrink: the tokens of every adapter are grouped (moe_group_kernel over tok_adapter; base
// tokens, adapter -1, fall in no group). Grid (rank groups of four, adapters), four warps; a warp takes
// eight tokens of its adapter at a time and computes 8 x 4 dot products per pass, so an A row is read
// once per eight tokens and an x row once per four ranks: tmp[t][j] = A[a][j] . x[t].
__global__ void lora_shrink_grouped_kernel(const float * __restrict__ a_stack, int r_max, int n_in, const int32_t * __restrict__ offsets,
                                           const int32_t * __restrict__ sorted, const float * __restrict__ x, int ldx,
                                           float * __restrict__ tmp) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int a = blockIdx.y, j0 = blockIdx.x * 4;
    const int begin = offsets[a], end = offsets[a + 1];
    const float * ar = a_stack + ((size_t)a * r_max + j0) * n_in;
    for (int p0 = begin + warp * 8; p0 < end; p0 += 8 * (blockDim.x >> 5)) {
        int tok[8];
        float acc[8][4];
#pragma unroll
        for (int tt = 0; tt < 8; ++tt) {
            tok[tt] = p0 + tt < end ? sorted[p0 + tt] : -1;
            acc[tt][0] = acc[tt][1] = acc[tt][2] = acc[tt][3] = 0.f;
        }
        for (int k = lane * 4; k < n_in; k += 128) {
            float4 av[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) av[r] = j0 + r < r_max ? *reinterpret_cast<const float4 *>(ar + (size_t)r * n_in + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                if (tok[tt] < 0) continue;
                const float4 xv = *reinterpret_cast<const float4 *>(x + (size_t)tok[tt] * ldx + k);
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[tt][r] += av[r].x * xv.x + av[r].y * xv.y + av[r].z * xv.z + av[r].w * xv.w;
            }
        }
#pragma unroll
        for (int tt = 0; tt < 8; ++tt) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float v = warp_sum(acc[tt][r]);
                if (lane == 0 && tok[tt] >= 0 && j0 + r < r_max) tmp[(size_t)tok[tt] * r_max + j0 + r] = v;
            }
        }
    }
}

__global__ void lora_expand_kernel(const float * __restrict__ b_stack, int r_max, int n_out, const float * __restrict__ scales,
                                   const int32_t * __restrict__ tok_adapter, const float * __restrict__ tmp, float * __restrict__ y, int ldy) {
    const int t = blockIdx.y;
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= n_out) return;
    const int a = tok_adapter[t];
    if (a < 0) return;
    const float * br = b_stack + ((size_t)a * n_out + o) * r_max;
    float acc = 0.f;
    for (int j = 0; j < r_max; ++j) acc += br[j] * tmp[(size_t)t * r_max + j];
    y[(size_t)t * ldy + o] += scales[a] * acc;
}

template <class F> void dispatch_type(uint32_t type, F && f) {
    switch (type) {
        case GGML_F32: f(std::integral_constant<uint32_t, GGML_F32>{}); break;
        case GGML_F16: f(std::integral_constant<uint32_t, GGML_F16>{}); break;
        case GGML_BF16: f(std::integral_constant<uint32_t, GGML_BF16>{}); break;
        case GGML_Q8_0: f(std::integral_constant<uint32_t, GGML_Q8_0>{}); break;
        case GGML_Q4_K: f(std::integral_constant<uint32_t, GGML_Q4_K>{}); break;
        case GGML_MXFP4: f(std::integral_constant<uint32_t, GGML_MXFP4>{}); break;
        default: break;
    }
}

} // namespace

void launch_pack(const RowDesc * rows, int n_rows, int n_tokens, const int32_t * block_table, int max_blocks, int block_tokens,
                 int tile_tokens, PackMaps maps, cudaStream_t stream) {
    pack_scan_kernel<<<1, 1024, 0, stream>>>(rows, n_rows, tile_tokens, maps.cu_rows, maps.out_rank, maps.tile_rank);
    pack_fill_kernel<<<(n_tokens + 255) / 256, 256, 0, stream>>>(rows, n_rows, n_tokens, block_table, max_blocks, block_tokens, tile_tokens, maps);
}

void launch_block_table_patch(int32_t * block_table, const int32_t * patches, int n_patches, cudaStream_t stream, int table_entries, int n_blocks,
                              int * check) {
    if (n_patches <= 0) return;
    block_table_patch_kernel<<<(n_patches + 255) / 256, 256, 0, stream>>>(block_table, patches, n_patches, table_entries, n_blocks, check);
}

void launch_kv_block_copy(KvLayout kv, int n_layer, const int32_t * pairs, int n_pairs, cudaStream_t stream) {
    if (n_pairs <= 0) return;
    kv_block_copy_kernel<<<dim3(n_pairs, n_layer), 256, 0, stream>>>(kv, n_layer, pairs);
}

void launch_kv_snapshot(KvLayout kv, int n_layer, const int32_t * table_row, int pos_first, int n_pos, void * dense, bool to_cache,
                        cudaStream_t stream) {
    if (n_pos <= 0) return;
    kv_snapshot_kernel<<<dim3(n_pos, n_layer * 2), 128, 0, stream>>>(kv, table_row, pos_first, static_cast<uint16_t *>(dense), n_pos, to_cache ? 1 : 0);
}

void launch_kv_quant_store(const float * qkv, int ld, int n_tokens, int n_head, KvLayout kv, int layer, const int32_t * tok_cell, cudaStream_t stream) {
    if (n_tokens <= 0) return;
    kv_quant_store_kernel<<<dim3(n_tokens), 256, 0, stream>>>(qkv, ld, n_head, kv, layer, tok_cell);
}

void launch_kv_dequant(KvLayout kv, int layer, int n_rows, int n_scratch_rows, int max_row_blocks, const int32_t * cu_rows, const int32_t * tok_slot,
                       const int32_t * tok_pos, const int32_t * tok_pos_min, int skip_tokens, cudaStream_t stream) {
    if (n_rows <= 0 || n_scratch_rows <= 0 || max_row_blocks <= 0) return;
    // grid.x: the rows that need the scratch; a row's CTAs walk its (block, K | V, head) units in strides of grid.y, a
    // handful of units each
    const int units = max_row_blocks * 2 * kv.n_head_kv;
    kv_dequant_kernel<<<dim3(n_scratch_rows, std::max(1, std::min(units / 4, 512))), 256, 0, stream>>>(kv, layer, n_rows, cu_rows, tok_slot, tok_pos,
                                                                                                      tok_pos_min, skip_tokens);
}

void launch_embed(WeightView embd, const int32_t * tokens, int n_tokens, float * x, cudaStream_t stream, int * check) {
    dispatch_type(embd.type, [&](auto tag) {
        embed_kernel<decltype(tag)::value><<<n_tokens, 128, 0, stream>>>(embd, tokens, x, check);
    });
}

void launch_rms_norm(const float * x, int ldx, const int32_t * gather, const float * w, int n, float eps, float * y, int ldy, int n_tokens,
                     cudaStream_t stream, const SplitAct * split) {
    const SplitAct sa = split && n % 32 == 0 ? *split : SplitAct{};
    const bool aligned = n % 32 == 0 && ldx % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) % 16 == 0 && x != y;
    if (aligned) launch_pdl(rms_norm4_kernel, dim3(n_tokens), dim3(256), 0, stream, x, ldx, gather, w, n, eps, y, ldy, sa);
    else launch_pdl(rms_norm_kernel, dim3(n_tokens), dim3(256), 0, stream, x, ldx, gather, w, n, eps, y, ldy, sa);
}

void launch_gemm_rows(WeightView w, const float * x, int ldx, int n_tokens, float * y, int ldy, const float * bias, const float * residual,
                      int ldr, cudaStream_t stream) {
    const int warps = 8;
    if (n_tokens <= 0 || w.n_out == 0) return;
    dispatch_type(w.type, [&](auto tag) {
        // the kernel strides over token groups, so a capped grid.x still covers every token
        const dim3 grid(std::min((n_tokens + 7) / 8, 1024), (w.n_out + warps - 1) / warps);
        gemm_rows_kernel<decltype(tag)::value><<<grid, warps * 32, 0, stream>>>(w, x, ldx, n_tokens, y, ldy, bias, residual, ldr);
    });
}

void launch_rope_store(float * qkv, int ld, int n_tokens, const RopeStoreArgs & a, cudaStream_t stream, const float * partial, int n_chunks,
                       int t_stride, int ld_partial, const float * bias) {
    launch_pdl(rope_store_kernel, dim3(n_tokens, (a.n_head + a.n_head_kv + 7) / 8), dim3(256), 0, stream, qkv, ld, a.n_head, a.n_head_kv, a.head_dim,
               a.n_rot, a.neox ? 1 : 0, a.inv_freq, a.tok_pos, a.tok_cell, a.kv, a.layer, partial, n_chunks, t_stride, ld_partial, bias);
}

// The partial-sum form reads and writes four columns at a time and relies on the rotation touching
// every q and k element's final value only after the block's own columns are formed.
bool rope_store_from_partial_supported(const RopeStoreArgs & a, const float * qkv, int ld, int n_out, const float * bias) {
    return a.head_dim % 4 == 0 && ld % 4 == 0 && (uintptr_t)qkv % 16 == 0 && (!bias || (uintptr_t)bias % 16 == 0) &&
           n_out == (a.n_head + 2 * a.n_head_kv) * a.head_dim && n_out % 4 == 0;
}

void launch_attention_ref(const float * qkv, int ld, int n_tokens, int n_head, KvLayout kv, int layer, const int32_t * tok_slot,
                          const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, cudaStream_t stream, const SplitAct * split) {
    const int warps = 4;
    attention_ref_kernel<<<dim3((n_head + warps - 1) / warps, n_tokens), warps * 32, 0, stream>>>(qkv, ld, n_head, kv, layer, tok_slot, tok_pos,
                                                                                                tok_pos_min, out, ldo, split && kv.head_dim % 32 == 0 ? *split : SplitAct{});
}

void launch_split_prep(const float * x, int ldx, int n, int n_tokens, const SplitAct & split, cudaStream_t stream, const int32_t * gather,
                       int gather_div) {
    if (n % 32 == 0 && ldx % 4 == 0 && (uintptr_t)x % 16 == 0)
        launch_pdl(split_prep4_kernel, dim3((n + 1023) / 1024, n_tokens), dim3(256), 0, stream, x, ldx, n, split, gather, gather_div);
    else
        launch_pdl(split_prep_kernel, dim3((n + 255) / 256, n_tokens), dim3(256), 0, stream, x, ldx, n, split, gather, gather_div);
}

void launch_swiglu(const float * gu, int ld, int ff, int n_tokens, float * h, int ldh, cudaStream_t stream, const SplitAct * split) {
    const SplitAct sa = split && ff % 32 == 0 ? *split : SplitAct{};
    const bool aligned = ff % 32 == 0 && ld % 4 == 0 && ldh % 4 == 0 && ((uintptr_t)gu | (uintptr_t)h) % 16 == 0;
    if (aligned) launch_pdl(swiglu4_kernel, dim3((ff + 1023) / 1024, n_tokens), dim3(256), 0, stream, gu, ld, ff, h, ldh, sa);
    else launch_pdl(swiglu_kernel, dim3((ff + 255) / 256, n_tokens), dim3(256), 0, stream, gu, ld, ff, h, ldh, sa);
}

void launch_moe_route(const float * router_logits, int n_expert, int k, int n_tokens, int32_t * ids, float * weights, cudaStream_t stream) {
    moe_route_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(router_logits, n_expert, k, n_tokens, ids, weights);
}

void launch_moe_group(const int32_t * pair_expert, int n_pairs, int n_expert, int32_t * offsets, int32_t * sorted, cudaStream_t stream) {
    moe_group_kernel<<<1, 1024, 0, stream>>>(pair_expert, n_pairs, n_expert, offsets, sorted);
}

void launch_moe_gemm_grouped(WeightView w_all, uint64_t expert_stride_bytes, int n_expert, const int32_t * offsets, const int32_t * sorted,
                             const float * x, int ldx, int x_div, float * y, int ldy, cudaStream_t stream) {
    const int warps = 8;
    dispatch_type(w_all.type, [&](auto tag) {
        moe_gemm_grouped_kernel<decltype(tag)::value><<<dim3((w_all.n_out + warps - 1) / warps, n_expert), warps * 32, 0, stream>>>(
            w_all, expert_stride_bytes, offsets, sorted, x, ldx, x_div, y, ldy);
    });
}

void launch_moe_combine(const float * y_pairs, int ld, const int32_t * ids, const float * weights, int k, int d, int n_tokens,
                        const float * residual, float * out, cudaStream_t stream) {
    moe_combine_kernel<<<dim3((d + 255) / 256, n_tokens), 256, 0, stream>>>(y_pairs, ld, ids, weights, k, d, residual, out);
}

void launch_lora_shrink(const float * a_stack, int r_max, int n_in, const int32_t * tok_adapter, const float * x, int ldx, int n_tokens,
                        float * tmp, cudaStream_t stream) {
    const int warps = 4;
    lora_shrink_kernel<<<dim3((r_max + warps - 1) / warps, n_tokens), warps * 32, 0, stream>>>(a_stack, r_max, n_in, tok_adapter, x, ldx, tmp);
}

void launch_lora_shrink_grouped(const float * a_stack, int r_max, int n_in, int n_adapters, const int32_t * offsets, const int32_t * sorted,
                                const float * x, int ldx, float * tmp, cudaStream_t stream) {
    lora_shrink_grouped_kernel<<<dim3((r_max + 3) / 4, n_adapters), 128, 0, stream>>>(a_stack, r_max, n_in, offsets, sorted, x, ldx, tmp);
}

void launch_lora_expand(const float * b_stack, int r_max, int n_out, const float * scales, const int32_t * tok_adapter, const float * tmp,
                        int n_tokens, float * y, int ldy, cudaStream_t stream) {
    lora_expand_kernel<<<dim3((n_out + 255) / 256, n_tokens), 256, 0, stream>>>(b_stack, r_max, n_out, scales, tok_adapter, tmp, y, ldy);
}

} // namespace rb200
