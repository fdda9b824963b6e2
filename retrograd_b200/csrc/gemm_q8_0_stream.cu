// Dequant-fused Q8_0 weight GEMM for decode steps of at most 8 tokens, on the skeleton of
// gemm_q4k_stream.cu: a CTA owns a K chunk of eight 256-column groups and a range of 16-row units,
// two warps share a group (one per 128 columns) and keep the activation fragments of THEIR columns in
// registers, every warp runs its own ring of bulk asynchronous copies (2176 bytes per stage: the
// unit's 16 x 4 block scales and 16 x 128 int8 weights), the tokens are the N = 8 dimension of
// mma.sync.m16n8k16, partial sums per K chunk are added in chunk order by the finish kernel.
//
// Exact arithmetic without per-weight instructions beyond placing bytes: the weight operand is the
// byte q + 128 (one XOR per four weights) put into the low byte of an f16, i.e. the exact value
// (q + 128) * 2^-24; the activations are hi + lo f16 pairs; a 32-column block is exactly two K steps,
// so its sum comes out of the MMAs on its own and gets, in f32,
//     d_block * (2^24 * sum - 128 * sum_of_x_over_the_block).
// The tile-major copy stores the weights in fragment order: what lane (g, tq) needs for four K steps
// of one row is 16 consecutive bytes, and a warp's load is 512 consecutive bytes.

#include "kernels.cuh"
#include "blocks.hpp"
#include "mma_common.cuh"
#include "tc5_common.cuh"

namespace rb200 {

namespace {

constexpr int SW = 8;                      // 256-column groups per K chunk
constexpr int NWARP = 2 * SW;
constexpr int STHREADS = NWARP * 32;
constexpr int STAGES = 4;
constexpr int UB = 2;                      // 16-row units per block-wide reduction
constexpr int STAGE_BYTES = (int)kQ8TileBytes;
constexpr int RED_BYTES = 2 * UB * NWARP * 128 * 4;
constexpr int RING_BYTES = NWARP * STAGES * STAGE_BYTES;
constexpr int SMEM_BYTES = RED_BYTES + RING_BYTES + NWARP * STAGES * 8 + 16;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

// grid (256-column groups, 16-row units), 128 threads: thread = (row of the unit, block of the group)
__global__ void q8_0_retile_kernel(const uint8_t * __restrict__ rows, uint32_t n_out, uint32_t n_sb, uint32_t row_bytes, uint8_t * __restrict__ tiled) {
    const uint32_t sb = blockIdx.x, unit = blockIdx.y;
    const uint32_t r = threadIdx.x >> 3, blk8 = threadIdx.x & 7;        // row 0..15, block 0..7 of the group
    const uint32_t kh = blk8 >> 2, blk = blk8 & 3;
    const uint32_t row = unit * 16 + r;
    uint8_t * dst = tiled + (((size_t)unit * n_sb + sb) * 2 + kh) * kQ8TileBytes;
    uint16_t d = 0;
    uint32_t q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (row < n_out) {
        const uint8_t * src = rows + (size_t)row * row_bytes + ((size_t)sb * 8 + blk8) * 34;
        d = *reinterpret_cast<const uint16_t *>(src);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = (uint32_t)src[2 + 4 * i] | (uint32_t)src[3 + 4 * i] << 8 | (uint32_t)src[4 + 4 * i] << 16 | (uint32_t)src[5 + 4 * i] << 24;
    }
    *reinterpret_cast<uint16_t *>(dst + (r * 4 + blk) * 2) = d;
    // word i of the block = columns 4 i .. 4 i + 3: K step 2 blk + i / 4 of the half, lane quarter tq = i % 4
    const uint32_t g = r & 7, rowsel = r >> 3;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t ks = 2 * blk + (i >> 2), tq = i & 3;
        const uint32_t kq = ks >> 2, ksl = ks & 3;
        *reinterpret_cast<uint32_t *>(dst + 128 + ((((kq * 2 + rowsel) * 8 + g) * 4 + tq) * 4 + ksl) * 4) = q[i];
    }
}

// PACK4: at most four tokens; MMA column t carries the hi term of token t, column t + 4 its lo term.
template <bool PACK4>
__global__ void __launch_bounds__(STHREADS, 1) gemm_q8_0_stream_kernel(const uint8_t * __restrict__ Wt, int n_in, int n_out, SplitAct X, int T,
                                                                       float * __restrict__ partial, int units_per_cta, int * __restrict__ error_flag) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    float * red = reinterpret_cast<float *>(smem_raw);                       // [2][UB][NWARP][128]
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t ring_base = smem_base + RED_BYTES;
    const uint32_t bar_base = ring_base + RING_BYTES;
    volatile int * abort_flag = reinterpret_cast<volatile int *>(smem_raw + RED_BYTES + RING_BYTES + NWARP * STAGES * 8);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int n_sb = n_in / 256, n_sub = n_in / 32;
    const int kchunk = blockIdx.y;
    const int sb = kchunk * SW + (warp >> 1);
    const int kh = warp & 1;
    const bool sb_valid = sb < n_sb;
    const int n_units = (n_out + 15) / 16;
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

    auto issue = [&](int u, int stage) {
        const uint8_t * src = Wt + (((size_t)u * n_sb + sb) * 2 + kh) * kQ8TileBytes;
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

    // ---- activation fragments of MMA column g, and -128 * (sum of x) per block for this lane's two result columns
    uint32_t bh[8][2], bl[8][2];
    float nsx[4][2];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) bh[ks][0] = bh[ks][1] = bl[ks][0] = bl[ks][1] = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) nsx[b][0] = nsx[b][1] = 0.f;
    {
        const int tok = PACK4 ? (g & 3) : g;
        if (sb_valid && tok < T) {
            const size_t row = (size_t)tok * X.ld + (size_t)sb * 256 + (size_t)kh * 128;
            const __half * src_a = (PACK4 && g >= 4) ? X.lo : X.hi;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                // K step ks = block ks / 2 of the half, columns (ks % 2) * 16 + 4 tq .. + 3 of the block
                const int e = (ks >> 1) * 32 + (ks & 1) * 16 + 4 * tq;
                const uint2 vh = *reinterpret_cast<const uint2 *>(src_a + row + e);
                bh[ks][0] = vh.x;      // elements 0, 1 -> K slots 2 tq, 2 tq + 1
                bh[ks][1] = vh.y;      // elements 2, 3 -> K slots 2 tq + 8, 2 tq + 9
                if (!PACK4) {
                    const uint2 vl = *reinterpret_cast<const uint2 *>(X.lo + row + e);
                    bl[ks][0] = vl.x;
                    bl[ks][1] = vl.y;
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = 2 * tq + e;
            const int t = col;                      // PACK4: columns >= 4 carry lo terms and take no offset
            if (sb_valid && t < T && (!PACK4 || col < 4)) {
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const size_t at = (size_t)t * n_sub + (size_t)sb * 8 + kh * 4 + b;
                    nsx[b][e] = -128.f * (__half2float(X.sum_hi[at]) + __half2float(X.sum_lo[at]));
                }
            }
        }
    }

    auto compute = [&](int stage, float (&part)[4]) {
        const uint8_t * base = smem_raw + RED_BYTES + (warp * STAGES + stage) * STAGE_BYTES;
        const uint2 sc0 = *reinterpret_cast<const uint2 *>(base + g * 8);            // four block scales of row g
        const uint2 sc1 = *reinterpret_cast<const uint2 *>(base + (g + 8) * 8);      // row g + 8
        float acc[4][4];
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f;
#pragma unroll
        for (int kq = 0; kq < 2; ++kq) {
            const uint4 wa = *reinterpret_cast<const uint4 *>(base + 128 + ((((kq * 2 + 0) * 8 + g) * 4 + tq) * 16));
            const uint4 wb = *reinterpret_cast<const uint4 *>(base + 128 + ((((kq * 2 + 1) * 8 + g) * 4 + tq) * 16));
            const uint32_t ra[4] = {wa.x, wa.y, wa.z, wa.w}, rb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int ksl = 0; ksl < 4; ++ksl) {
                const int ks = kq * 4 + ksl, b = ks >> 1;
                const uint32_t ua = ra[ksl] ^ 0x80808080u, ub = rb[ksl] ^ 0x80808080u;      // q + 128 per byte
                const uint32_t a0 = __byte_perm(ua, 0u, 0x4140), a2 = __byte_perm(ua, 0u, 0x4342);
                const uint32_t a1 = __byte_perm(ub, 0u, 0x4140), a3 = __byte_perm(ub, 0u, 0x4342);
                mma_f16(acc[b], a0, a1, a2, a3, bh[ks][0], bh[ks][1]);
                if (!PACK4) mma_f16(acc[b], a0, a1, a2, a3, bl[ks][0], bl[ks][1]);
            }
        }
        const __half2 s0a = *reinterpret_cast<const __half2 *>(&sc0.x), s0b = *reinterpret_cast<const __half2 *>(&sc0.y);
        const __half2 s1a = *reinterpret_cast<const __half2 *>(&sc1.x), s1b = *reinterpret_cast<const __half2 *>(&sc1.y);
        const float d0[4] = {__low2float(s0a), __high2float(s0a), __low2float(s0b), __high2float(s0b)};
        const float d1[4] = {__low2float(s1a), __high2float(s1a), __low2float(s1b), __high2float(s1b)};
        part[0] = part[1] = part[2] = part[3] = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            part[0] += d0[b] * fmaf(acc[b][0], 16777216.f, nsx[b][0]);
            part[1] += d0[b] * fmaf(acc[b][1], 16777216.f, nsx[b][1]);
            part[2] += d1[b] * fmaf(acc[b][2], 16777216.f, nsx[b][0]);
            part[3] += d1[b] * fmaf(acc[b][3], 16777216.f, nsx[b][1]);
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
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            if (work && alive) compute(stage, part);
            *reinterpret_cast<float4 *>(&red[((buf * UB + j) * NWARP + warp) * 128 + lane * 4]) = make_float4(part[0], part[1], part[2], part[3]);
            if (work) {
                __syncwarp();       // every lane has read the stage before it is refilled
                if (lane == 0 && alive && u + STAGES < u_end) issue(u + STAGES, stage);
                ++it;
            }
        }
        __syncthreads();
        // add the sixteen warps' contributions in warp order: one thread per (unit of the batch, fragment slot)
        if (tid < UB * 128) {
            const int j = tid >> 7, v = tid & 127;
            const int u = ub + j;
            const int ln = v >> 2, e = v & 3;
            const int t = 2 * (ln & 3) + (e & 1);
            if (u < u_end && t < T) {
                const float * src = &red[(buf * UB + j) * NWARP * 128 + v];
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < NWARP; ++w) sum += src[w * 128];
                if (PACK4) {       // the lo terms sit four MMA columns to the right: lane tq + 2
                    float lo = 0.f;
#pragma unroll
                    for (int w = 0; w < NWARP; ++w) lo += src[w * 128 + 8];
                    sum += lo;
                }
                const int o = u * 16 + (ln >> 2) + ((e >> 1) << 3);
                if (o < n_out) partial[((size_t)kchunk * 8 + t) * n_out + o] = sum;
            }
        }
        buf ^= 1;
    }
    if (!alive || *abort_flag) {
        if (lane == 0) {
            atomicExch(error_flag, 1);
            if (sb_valid) {
                const long long start = clock64();
                for (int s2 = 0; s2 < STAGES; ++s2) {
                    const int consumed = (it + STAGES - 1 - s2) / STAGES;
                    while (!tc5::mbar_try_wait(my_bars + s2 * 8, consumed & 1) && clock64() - start < (1ll << 28)) {}
                }
            }
        }
    }
}

} // namespace

void launch_q8_0_retile(const uint8_t * rows, uint32_t n_out, uint32_t n_in, uint32_t row_bytes, uint8_t * tiled, cudaStream_t stream) {
    q8_0_retile_kernel<<<dim3(n_in / 256, (n_out + 15) / 16), 128, 0, stream>>>(rows, n_out, n_in / 256, row_bytes, tiled);
}

bool gemm_q8_0_stream_supported(const WeightView & w, const SplitAct & x, int n_tokens) {
    return w.type == GGML_Q8_0 && w.tiled && w.n_in % 256 == 0 && x.hi && x.ld == (int)w.n_in && n_tokens >= 1 && n_tokens <= 8;
}

void launch_gemm_q8_0_stream(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                             const float * residual, int ldr, float * scratch, int n_sm, int * error_flag, cudaStream_t stream,
                             const FinishTail * tail) {
    const int n_sb = (int)w.n_in / 256;
    const int n_chunks = (n_sb + SW - 1) / SW;
    const int n_units = ((int)w.n_out + 15) / 16;
    static PerDeviceOnce configured;   // function attributes are per device
    if (configured.first()) {
        cudaFuncSetAttribute(gemm_q8_0_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaFuncSetAttribute(gemm_q8_0_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    }
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
    if (n_tokens <= 4) cudaLaunchKernelEx(&cfg, gemm_q8_0_stream_kernel<true>, w.tiled, (int)w.n_in, (int)w.n_out, x, n_tokens, scratch, units_per_cta, error_flag);
    else cudaLaunchKernelEx(&cfg, gemm_q8_0_stream_kernel<false>, w.tiled, (int)w.n_in, (int)w.n_out, x, n_tokens, scratch, units_per_cta, error_flag);
    launch_gemm_stream_finish(scratch, n_chunks, (int)w.n_out, n_tokens, 8, y, ldy, bias, residual, ldr, stream, tail);
}

} // namespace rb200
