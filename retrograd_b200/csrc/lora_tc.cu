// Segmented multi-adapter LoRA on the tensor cores: y[t] += scale[a(t)] * B[a(t)] (A[a(t)] x[t]) for the
// tokens of a step whose rows name different adapters (reference: per-row adapters of the batched step,
// crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:2539-2564, 2987-3006).
//
// The step's tokens are grouped by adapter once (offsets / sorted, built by the grouping kernel); a
// segment is cut into tiles of 16 tokens, and each tile is one m16n8k8 TF32 MMA row block:
//   shrink: tile [16 tokens x n_in] times A[a]^T [n_in x r]      -> tmp[split][t][r]   (K split over grid.y)
//   expand: tile [16 tokens x r]    times B[a]^T [r x n_out]     -> y[t][o] += scale[a] * ...
// Both operands are F32 in memory. Every value is split v = big + small with both parts TF32, and a product
// is accumulated as big*small + small*big + big*big in F32, which keeps the result within a few units of
// 2^-22 of the F32 product the CPU path computes; the K order inside an MMA is free, so a thread's four
// consecutive columns (one 16-byte load) feed two MMAs directly.
//
// The partial results of the K splits are summed by the expand kernel in split order, and a token's row
// is produced by exactly one tile: results do not depend on which other rows share the step.
// Targets that read the same input rows (q, k, v; gate, up) go through ONE pair of launches (grid.z = target):
// the kernels are bound by launch and load latency, not by their bytes.
#include "kernels.cuh"

namespace rb200 {

namespace {

__device__ __forceinline__ void split_tf32(float v, uint32_t & big, uint32_t & small) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(big) : "f"(v));
    const float rest = v - __uint_as_float(big);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(small) : "f"(rest));
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// three TF32 MMAs for one F32-accurate 16 x 8 x 8 product: the small cross terms first
__device__ __forceinline__ void mma_3x(float (&c)[4], const uint32_t (&ab)[4], const uint32_t (&as)[4], uint32_t bb0, uint32_t bb1, uint32_t bs0,
                                       uint32_t bs1) {
    mma_tf32(c, ab[0], ab[1], ab[2], ab[3], bs0, bs1);
    mma_tf32(c, as[0], as[1], as[2], as[3], bb0, bb1);
    mma_tf32(c, ab[0], ab[1], ab[2], ab[3], bb0, bb1);
}

// The (adapter, 16-token tile) a CTA owns: tiles are numbered segment by segment. False past the last tile.
// The segment offsets are fetched by the whole CTA at once (one load latency instead of one per adapter).
constexpr int kMaxAdapters = 1024;
__device__ __forceinline__ bool find_tile(int tile, int n_adapters, const int32_t * __restrict__ offsets, int * sh_offsets, int & adapter, int & first,
                                          int & end) {
    for (int i = threadIdx.x; i <= n_adapters; i += blockDim.x) sh_offsets[i] = offsets[i];
    __syncthreads();
    for (int a = 0; a < n_adapters; ++a) {
        const int b = sh_offsets[a], e = sh_offsets[a + 1];
        const int n = (e - b + 15) >> 4;
        if (tile < n) {
            adapter = a;
            first = b + tile * 16;
            end = e;
            return true;
        }
        tile -= n;
    }
    return false;
}

// grid (tile bound, K splits), 8 warps: the warps take the CTA's columns in interleaved chunks of 16 and their
// 16 x (8 NR) partial results are added in warp order through shared memory. The work is a few hundred KB per
// launch, so the kernel is built for load parallelism: many short K ranges, four chunks' loads in flight per warp.
constexpr int kShrinkWarps = 8;
template <int NR>
__global__ void __launch_bounds__(kShrinkWarps * 32) lora_shrink_tc_kernel(const LoraGroup group, int r_max, int n_in, int n_adapters,
                                                             const int32_t * __restrict__ offsets, const int32_t * __restrict__ sorted,
                                                             const float * __restrict__ x, int ldx, float * __restrict__ tmp, int n_tokens,
                                                             int k_per_split) {
    // blockIdx.z: which of the group's targets (they share the input rows); each has its own region of tmp
    const float * __restrict__ a_stack = group.a[blockIdx.z];
    tmp += (size_t)blockIdx.z * gridDim.y * n_tokens * r_max;
    __shared__ float red[kShrinkWarps][16][NR * 8 + 1];
    __shared__ int sh_offsets[kMaxAdapters + 1];
    int adapter, first, end;
    if (!find_tile(blockIdx.x, n_adapters, offsets, sh_offsets, adapter, first, end)) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int tok0 = first + g < end ? sorted[first + g] : -1, tok1 = first + g + 8 < end ? sorted[first + g + 8] : -1;
    const float * x0 = x + (size_t)max(tok0, 0) * ldx + 4 * t;
    const float * x1 = x + (size_t)max(tok1, 0) * ldx + 4 * t;
    const float * ar = a_stack + ((size_t)adapter * r_max + g) * n_in + 4 * t;
    const int k0 = blockIdx.y * k_per_split, k1 = min(n_in, k0 + k_per_split);
    float acc[NR][4];
#pragma unroll
    for (int j = 0; j < NR; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int k = k0 + warp * 16; k < k1; k += kShrinkWarps * 16) {
        const float4 v0 = tok0 >= 0 ? *reinterpret_cast<const float4 *>(x0 + k) : zero;
        const float4 v1 = tok1 >= 0 ? *reinterpret_cast<const float4 *>(x1 + k) : zero;
        float4 av[NR];
#pragma unroll
        for (int j = 0; j < NR; ++j) av[j] = j * 8 + g < r_max ? *reinterpret_cast<const float4 *>(ar + (size_t)j * 8 * n_in + k) : zero;
        uint32_t pb[4], ps[4], qb[4], qs[4];      // the chunk's columns 4t, 4t+1 (first MMA) and 4t+2, 4t+3 (second)
        split_tf32(v0.x, pb[0], ps[0]);
        split_tf32(v1.x, pb[1], ps[1]);
        split_tf32(v0.y, pb[2], ps[2]);
        split_tf32(v1.y, pb[3], ps[3]);
        split_tf32(v0.z, qb[0], qs[0]);
        split_tf32(v1.z, qb[1], qs[1]);
        split_tf32(v0.w, qb[2], qs[2]);
        split_tf32(v1.w, qb[3], qs[3]);
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            uint32_t b0, s0, b1, s1;
            split_tf32(av[j].x, b0, s0);
            split_tf32(av[j].y, b1, s1);
            mma_3x(acc[j], pb, ps, b0, b1, s0, s1);
            split_tf32(av[j].z, b0, s0);
            split_tf32(av[j].w, b1, s1);
            mma_3x(acc[j], qb, qs, b0, b1, s0, s1);
        }
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        red[warp][g][j * 8 + 2 * t] = acc[j][0];
        red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
        red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
        red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    float * out = tmp + (size_t)blockIdx.y * n_tokens * r_max;
    for (int i = threadIdx.x; i < 16 * NR * 8; i += kShrinkWarps * 32) {
        const int row = i / (NR * 8), col = i % (NR * 8);
        if (first + row >= end || col >= r_max) continue;
        float v = red[0][row][col];
#pragma unroll
        for (int w = 1; w < kShrinkWarps; ++w) v += red[w][row][col];
        out[(size_t)sorted[first + row] * r_max + col] = v;
    }
}

// grid (tile bound, column groups of 128), 4 warps: a warp takes four column tiles of eight, with every load of
// the four (B rows and the y values they update) issued before the first MMA.
template <int NR>
__global__ void __launch_bounds__(128) lora_expand_tc_kernel(const LoraGroup group, int r_max, const float * __restrict__ scales,
                                                             int n_adapters, const int32_t * __restrict__ offsets, const int32_t * __restrict__ sorted,
                                                             const float * __restrict__ tmp, int n_splits, int n_tokens, float * __restrict__ y, int ldy,
                                                             int groups_per_cta, int vec2) {
    const int n_out = group.n_out[blockIdx.z];
    if ((int)blockIdx.y * groups_per_cta * 128 >= n_out) return;       // the grid's column groups cover the widest target
    const float * __restrict__ b_stack = group.b[blockIdx.z];
    tmp += (size_t)blockIdx.z * n_splits * n_tokens * r_max;
    y += group.y_offset[blockIdx.z];
    __shared__ int sh_offsets[kMaxAdapters + 1];
    int adapter, first, end;
    if (!find_tile(blockIdx.x, n_adapters, offsets, sh_offsets, adapter, first, end)) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int tok0 = first + g < end ? sorted[first + g] : -1, tok1 = first + g + 8 < end ? sorted[first + g + 8] : -1;
    // the tile's shrink results (K splits added in split order) as the A operand, split once
    uint32_t ab[NR][4], as[NR][4];
#pragma unroll
    for (int kk = 0; kk < NR; ++kk) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int tok = (e & 1) ? tok1 : tok0, r = kk * 8 + t + ((e & 2) ? 4 : 0);
            float v = 0.f;
            if (tok >= 0 && r < r_max)
                for (int s = 0; s < n_splits; ++s) v += tmp[((size_t)s * n_tokens + tok) * r_max + r];
            split_tf32(v, ab[kk][e], as[kk][e]);
        }
    }
    const float scale = scales[adapter];
    const float * br = b_stack + (size_t)adapter * n_out * r_max;
    constexpr int CT = 4;                          // column tiles per warp and column group
    struct Operands {
        float bv[CT][NR][2];
        float2 y0[CT], y1[CT];
    };
    // column group cg of this CTA: 128 columns, 32 per warp. Every load of a group is issued before its first MMA,
    // and the next group's loads before this group's MMAs (the CTA's prologue - tile lookup, token ids, the shrink
    // results - is paid once for `groups_per_cta` groups instead of once per group).
    auto o_base_of = [&](int cg) { return ((int)blockIdx.y * groups_per_cta + cg) * 128 + warp * (CT * 8); };
    auto load = [&](int cg, Operands & op) {
        const int o_base = o_base_of(cg);
#pragma unroll
        for (int i = 0; i < CT; ++i) {
            const int o0 = o_base + i * 8;
            const bool row_ok = o0 + g < n_out;
            const float * bo = br + (size_t)(o0 + g) * r_max;
#pragma unroll
            for (int kk = 0; kk < NR; ++kk) {
                const int r0 = kk * 8 + t, r1 = r0 + 4;
                op.bv[i][kk][0] = row_ok && r0 < r_max ? bo[r0] : 0.f;
                op.bv[i][kk][1] = row_ok && r1 < r_max ? bo[r1] : 0.f;
            }
            const int col = o0 + 2 * t;
            op.y0[i] = op.y1[i] = make_float2(0.f, 0.f);
            if (vec2 && col + 1 < n_out) {
                if (tok0 >= 0) op.y0[i] = *reinterpret_cast<const float2 *>(y + (size_t)tok0 * ldy + col);
                if (tok1 >= 0) op.y1[i] = *reinterpret_cast<const float2 *>(y + (size_t)tok1 * ldy + col);
            } else {
                if (tok0 >= 0 && col < n_out) op.y0[i].x = y[(size_t)tok0 * ldy + col];
                if (tok0 >= 0 && col + 1 < n_out) op.y0[i].y = y[(size_t)tok0 * ldy + col + 1];
                if (tok1 >= 0 && col < n_out) op.y1[i].x = y[(size_t)tok1 * ldy + col];
                if (tok1 >= 0 && col + 1 < n_out) op.y1[i].y = y[(size_t)tok1 * ldy + col + 1];
            }
        }
    };
    auto finish = [&](int cg, Operands & op) {
        const int o_base = o_base_of(cg);
#pragma unroll
        for (int i = 0; i < CT; ++i) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kk = 0; kk < NR; ++kk) {
                uint32_t b0, s0, b1, s1;
                split_tf32(op.bv[i][kk][0], b0, s0);
                split_tf32(op.bv[i][kk][1], b1, s1);
                mma_3x(c, ab[kk], as[kk], b0, b1, s0, s1);
            }
            const int col = o_base + i * 8 + 2 * t;
            op.y0[i].x += scale * c[0];
            op.y0[i].y += scale * c[1];
            op.y1[i].x += scale * c[2];
            op.y1[i].y += scale * c[3];
            if (vec2 && col + 1 < n_out) {
                if (tok0 >= 0) *reinterpret_cast<float2 *>(y + (size_t)tok0 * ldy + col) = op.y0[i];
                if (tok1 >= 0) *reinterpret_cast<float2 *>(y + (size_t)tok1 * ldy + col) = op.y1[i];
            } else {
                if (tok0 >= 0 && col < n_out) y[(size_t)tok0 * ldy + col] = op.y0[i].x;
                if (tok0 >= 0 && col + 1 < n_out) y[(size_t)tok0 * ldy + col + 1] = op.y0[i].y;
                if (tok1 >= 0 && col < n_out) y[(size_t)tok1 * ldy + col] = op.y1[i].x;
                if (tok1 >= 0 && col + 1 < n_out) y[(size_t)tok1 * ldy + col + 1] = op.y1[i].y;
            }
        }
    };
    // groups of this CTA that start inside the target's columns
    const int first_col = (int)blockIdx.y * groups_per_cta * 128;
    const int n_groups = min(groups_per_cta, (n_out - first_col + 127) / 128);
    Operands even, odd;
    load(0, even);
    for (int cg = 0; cg < n_groups; cg += 2) {
        if (cg + 1 < n_groups) load(cg + 1, odd);
        finish(cg, even);
        if (cg + 1 < n_groups) {
            if (cg + 2 < n_groups) load(cg + 2, even);
            finish(cg + 1, odd);
        }
    }
}

template <class F> void dispatch_rank_tiles(int r_max, F && f) {
    const int tiles = (r_max + 7) / 8;
    if (tiles <= 1) f(std::integral_constant<int, 1>{});
    else if (tiles <= 2) f(std::integral_constant<int, 2>{});
    else if (tiles <= 4) f(std::integral_constant<int, 4>{});
    else f(std::integral_constant<int, 8>{});
}

} // namespace

int lora_tc_splits(int n_in) {
    static const int k_per_split = [] { const char * e = std::getenv("RB200_LORA_SPLIT_K"); return e && std::atoi(e) >= 64 ? std::atoi(e) : 512; }();
    return std::max(1, std::min(kLoraTcMaxSplits, n_in / k_per_split));
}

bool lora_tc_supported(int r_max, int n_in, const float * a_stack, const float * x, int ldx) {
    return r_max >= 1 && r_max <= 64 && n_in % 16 == 0 && ldx % 4 == 0 && (uintptr_t)a_stack % 16 == 0 && (uintptr_t)x % 16 == 0;
}

void launch_lora_tc(const LoraGroup & group, const float * scales, int r_max, int n_in, int n_adapters, const int32_t * offsets, const int32_t * sorted,
                    const float * x, int ldx, int n_tokens, float * tmp, float * y, int ldy, cudaStream_t stream) {
    if (n_tokens <= 0 || n_adapters <= 0 || group.n <= 0) return;
    const int tiles = (n_tokens + 15) / 16 + n_adapters;          // every segment may end in a partial tile
    const int splits = lora_tc_splits(n_in);
    const int k_per_split = ((n_in + splits - 1) / splits + 15) / 16 * 16;
    int widest = 0, vec2 = ldy % 2 == 0 && (uintptr_t)y % 8 == 0 ? 1 : 0;
    for (int i = 0; i < group.n; ++i) {
        widest = std::max(widest, group.n_out[i]);
        if (group.y_offset[i] % 2 != 0) vec2 = 0;
    }
    dispatch_rank_tiles(r_max, [&](auto tag) {
        constexpr int NR = decltype(tag)::value;
        lora_shrink_tc_kernel<NR><<<dim3(tiles, splits, group.n), kShrinkWarps * 32, 0, stream>>>(group, r_max, n_in, n_adapters, offsets, sorted, x, ldx, tmp,
                                                                                                n_tokens, k_per_split);
        // column groups of 128 per CTA: as many as still leave a few waves of CTAs (a CTA's prologue is the larger part
        // of a one-group CTA's life)
        static const int forced = [] { const char * e = std::getenv("RB200_LORA_GROUPS_PER_CTA"); return e ? std::atoi(e) : 0; }();
        const int groups = (widest + 127) / 128;
        const int groups_per_cta = forced > 0 ? forced : std::max(1, std::min(8, tiles * groups * group.n / 600));
        lora_expand_tc_kernel<NR><<<dim3(tiles, (groups + groups_per_cta - 1) / groups_per_cta, group.n), 128, 0, stream>>>(
            group, r_max, scales, n_adapters, offsets, sorted, tmp, splits, n_tokens, y, ldy, groups_per_cta, vec2);
    });
}

} // namespace rb200
