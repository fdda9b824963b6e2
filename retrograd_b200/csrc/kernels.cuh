// Device-side views and launch wrappers of the decode step's kernels.
#pragma once

#include <cstdlib>

#include <cstdint>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

namespace rb200 {

// A weight matrix in device memory in its GGUF storage layout: n_out rows of n_in elements.
struct WeightView {
    const uint8_t * data = nullptr;
    uint32_t type = 0;
    uint32_t n_in = 0;
    uint32_t n_out = 0;
    uint32_t row_bytes = 0;
    // Q4_K, optional: the same blocks in the tile-major layout described at kQ4kTileBytes, rows
    // zero-padded to a multiple of 128 (read by the tcgen05 kernel and the weight-streaming kernel).
    // Q8_0, optional: the layout described at kQ8TileBytes, rows padded to a multiple of 16.
    const uint8_t * tiled = nullptr;
    // The matrix passed the host-side check its tcgen05 kernel needs, made once when the weights are uploaded.
    // Q4_K: every super-block lets the kernel fold the minimum term into the main accumulator (q4k_min_fold_ok).
    // Q8_0: every block scale keeps d * q inside the f16 range, so a weight is an exact f16 pair (q8_0_products_fit_f16).
    bool tc5_exact = false;
};

// Tile-major copy of a Q4_K matrix: one 18432-byte tile per (128 rows, 256-column super-block), tiles
// of a row tile consecutive over the super-blocks. A tile is four 4608-byte quarters of 32 rows. A
// quarter holds, for its rows, the 32 nibble bytes of 64-column groups 0 and 1 (2 x 1024 bytes), then
// the 32 block headers of 16 bytes (d, dmin, packed scales), then groups 2 and 3: either half of the
// columns together with the headers is one contiguous 2560-byte range, and a warp that takes one row
// per lane reads consecutive bytes.
constexpr size_t kQ4kTileBytes = 18432;
constexpr size_t kQ4kQuarterBytes = 4608;
__host__ __device__ inline size_t q4k_tile_hdr_offset(int p) { return (size_t)(p >> 5) * kQ4kQuarterBytes + 2048 + (size_t)(p & 31) * 16; }
__host__ __device__ inline size_t q4k_tile_group_offset(int p, int r) {
    return (size_t)(p >> 5) * kQ4kQuarterBytes + (size_t)r * 1024 + (r >= 2 ? 512 : 0) + (size_t)(p & 31) * 32;
}
inline size_t q4k_tiled_bytes(uint32_t n_out, uint32_t n_in) { return (size_t)((n_out + 127) / 128) * (n_in / 256) * kQ4kTileBytes; }
// Regroups GGUF-layout Q4_K rows into the tiled layout (device to device).
void launch_q4k_retile(const uint8_t * rows, uint32_t n_out, uint32_t n_in, uint32_t row_bytes, uint8_t * tiled, cudaStream_t stream);

// Tile-major copy of an MXFP4 expert bank: one 4352-byte tile per (expert, 128 rows, 64 columns), tiles of a row
// tile consecutive over the column groups: the rows' 32 nibble bytes (row p at 32 p), then their two E8M0 bytes.
constexpr size_t kMxfp4TileBytes = 4352;
size_t mxfp4_tiled_bytes(uint32_t n_expert, uint32_t n_out, uint32_t n_in);
// Regroups a GGUF-layout MXFP4 bank [expert][row][blocks of 17 bytes] into the tiled layout (device to device).
void launch_mxfp4_retile(const uint8_t * bank, uint32_t n_expert, uint32_t n_out, uint32_t n_in, uint8_t * tiled, cudaStream_t stream);
// Whether every block's E8M0 byte is in 104..128, i.e. every weight of the bank is an f16 (host memory).
bool mxfp4_scales_are_f16(const uint8_t * blocks, size_t n_blocks);
// Whether the driver offers tensor-map encoding (the TMA descriptors of the activation operands).
bool tensor_maps_available();

#ifdef __CUDACC__
// Kernel function attributes (the opt-in to more than 48 KB of dynamic shared memory) belong to a
// device, not to the process: first() is true the first time it is called with a given device current.
struct PerDeviceOnce {
    std::atomic<uint64_t> done[4] = {};
    bool first() {
        int device = 0;
        cudaGetDevice(&device);
        const uint64_t bit = 1ull << (device & 63);
        return (done[(device >> 6) & 3].fetch_or(bit) & bit) == 0;
    }
};

// Programmatic dependent launch. A kernel launched with launch_pdl() may be scheduled while the
// stream's previous kernel is still running; it must execute pdl_wait() before it reads or writes
// anything an earlier kernel of the stream touches (the wait returns when the previous kernel has
// completed and its writes are visible; without the launch attribute it is a no-op). pdl_trigger()
// tells the scheduler that the kernels launched after this one may be scheduled from now on. Every
// kernel launched this way executes pdl_wait() on every path, so completion stays transitive
// along the stream.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

// RB200_PDL=0: the kernels launched through launch_pdl() are serialised like plain launches.
inline bool pdl_enabled() {
    static const bool on = [] {
        const char * env = std::getenv("RB200_PDL");
        return !(env && env[0] == '0');
    }();
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// The bounds-checked build (-DRETRO_B200_CHECKED, libretro_b200_checked.so). Every index a kernel takes from
// device memory - a token id, a slot, a position, a block-table entry, a physical block id, an adapter index -
// is compared with its range before it is used. The first violation is recorded in the engine's check word
// {code, value, limit, count} and the access it would have addressed is skipped; the step then returns -1 with
// the word spelled out. It stands in for a memory checker on machines where none can be run. In the normal
// build RB_CHECK compiles to nothing and the `check` pointers below stay null.
enum CheckCode : int { CHECK_OK = 0, CHECK_TOKEN = 1, CHECK_SLOT = 2, CHECK_POSITION = 3, CHECK_TABLE_INDEX = 4, CHECK_BLOCK = 5, CHECK_CELL = 6, CHECK_ADAPTER = 7 };
#ifdef __CUDACC__
#ifdef RETRO_B200_CHECKED
__device__ __forceinline__ bool rb_check_in_range(int * word, int code, long long value, long long limit) {
    if (value >= 0 && value < limit) return true;
    if (word) {
        if (atomicCAS(word, 0, code) == 0) {
            word[1] = (int)value;
            word[2] = (int)limit;
        }
        atomicAdd(word + 3, 1);
    }
    return false;
}
#define RB_CHECK(word, code, value, limit, on_fail)                              \
    do {                                                                         \
        if (!rb_check_in_range((word), (code), (long long)(value), (long long)(limit))) { on_fail; } \
    } while (0)
#else
#define RB_CHECK(word, code, value, limit, on_fail) do { } while (0)
#endif
#endif

// An activation matrix [t][ld] prepared for the exact tensor-core GEMM: the two-term f16 split
// x = hi + lo, and per 32-element sub-block the sum of x, again as hi + lo ([t][ld / 32]).
struct SplitAct {
    __half * hi = nullptr;
    __half * lo = nullptr;
    __half * sum_hi = nullptr;
    __half * sum_lo = nullptr;
    int ld = 0;
    int has_maps = 0;
    // TMA descriptors over hi and lo ([rows][ld] f16, boxes of 64 columns x 128 rows, 128-byte swizzle)
    alignas(64) CUtensorMap map_hi;
    alignas(64) CUtensorMap map_lo;
};

// Fills the TMA descriptors of `s` for `rows` rows; returns false when the driver entry point is
// unavailable (the kernels that need them are then not selected).
bool split_act_encode_maps(SplitAct & s, size_t rows);

// The step of the layer that consumes a streaming GEMM's result, done by the GEMM's finish kernel on the
// row it has just summed (one launch and one pass over the row less):
//   kind 1: y is written, then RMS-normalised with `norm_w` into `out` (f32, may be null) and `split`;
//   kind 2: the row is [gate | up], two halves of n_out / 2 columns: silu(gate) * up goes to `out`
//           (may be null) and `split`; y itself is not written.
//   kind 3: the row is a token's [q | k | v]: y is written, q and k are rotated in place and k, v
//           stored into the paged cache (`rope`; y, ldy and the token count come from the GEMM).
// The arithmetic and its order are those of the separate kernels, so results do not depend on the fusion.
struct RopeStoreArgs;
struct FinishTail {
    int kind = 0;
    const RopeStoreArgs * rope = nullptr;
    const float * norm_w = nullptr;
    float eps = 0.f;
    float * out = nullptr;
    int ld_out = 0;
    SplitAct split{};
};
bool finish_tail_supported(const FinishTail & tail, int n_out, const float * y, int ldy, const float * bias, const float * residual, int ldr);

// One row of a step plan as the packing kernel reads it (32 bytes).
struct RowDesc {
    int32_t slot;
    int32_t n;
    int32_t pos0;
    int32_t sample;     // 0/1
    int32_t adapter;    // stacked adapter index, -1 = none
    int32_t pos_min;    // first resident position of the slot once this step is applied
    int32_t pad0;
    int32_t pad1;
};

// Per sampling row parameters (64 bytes).
struct SampleDesc {
    float temperature;
    float top_p;
    int32_t top_k;        // <= 0 disabled
    float min_p;          // <= 0 disabled
    uint32_t seed;
    uint32_t draw_lo;     // per-request draw counter
    uint32_t draw_hi;
    uint32_t n_top;       // top logprobs requested
    uint32_t flags;       // bit0: v2 row (post-transform reporting), bit1: want sampled_logprob, bit2: greedy without edits
    uint32_t edit_begin;  // range in the logit-edit list
    uint32_t edit_end;
    uint32_t pad[5];      // pad[0]: 1 + word offset of the row's grammar mask (0: none); pad[1]: 1 + the token a reasoning budget forces (0: none)
};

// One sparse change of a logits row before sampling (v2 rows): logit_bias adds, penalties.
struct LogitEdit {
    int32_t id;
    float bias;        // added first
    float repeat;      // repeat penalty (1 = none): multiplies non-positive, divides positive logits
    float subtract;    // count * frequency + presence
};

struct SampleOut {
    int32_t token;
    float logprob;           // temperature-1 logprob of token under the raw logits
    float sampled_logprob;   // post-transformation logprob (v2 + want_logprob)
    uint32_t n_top;
};

// Batch maps the packing kernel writes.
struct PackMaps {
    int32_t * cu_rows;     // [R + 1]
    int32_t * out_rank;    // [R + 1] exclusive scan of sample flags
    int32_t * tok_slot;    // [T]
    int32_t * tok_pos;     // [T]
    int32_t * tok_row;     // [T]
    int32_t * tok_cell;    // [T] physical KV cell = block * block_tokens + offset
    int32_t * tok_adapter; // [T]
    int32_t * tok_pos_min; // [T]
    int32_t * out_index;   // [S]
    int32_t * tile_rank;   // [R + 1] exclusive scan of the rows' attention tile counts
    int2 * attn_items;     // [sum of tiles] (first token index, tokens in the tile)
    // ranges for the bounds-checked build
    int32_t n_slots = 0, n_blocks = 0, n_adapters = 0;
    int * check = nullptr;
};

// Storage types of the KV pool. F16: the pool is what the attention kernels read. Q8_0 / Q4_0 (ggml's block formats:
// per 32 elements an f16 scale and 32 int8, or 16 bytes of nibble pairs): the pool holds `q_row_bytes` per (block,
// head, cell) - the row's quants, then its scales - and `k` / `v` point to a one-layer f16 scratch with the pool's
// block numbering (`layer_stride` 0) that kv_dequant fills, per layer, for the sequences of the step.
enum KvStorage : int32_t { KV_F16 = 0, KV_Q8_0 = 1, KV_Q4_0 = 2 };

struct KvLayout {
    __half * k;            // [n_blocks][n_head_kv][block_tokens][head_dim] per layer, layers consecutive
    __half * v;
    uint64_t layer_stride; // elements per layer
    uint8_t * kq = nullptr;      // quantised pool: [n_blocks][n_head_kv][block_tokens][q_row_bytes] per layer
    uint8_t * vq = nullptr;
    uint64_t q_layer_stride = 0; // bytes per layer
    int32_t storage = KV_F16;
    int32_t q_row_bytes = 0;
    int32_t n_head_kv;
    int32_t head_dim;
    int32_t block_tokens;
    const int32_t * block_table;  // [n_slots][max_blocks]
    int32_t max_blocks;
    // ranges for the bounds-checked build
    int32_t n_blocks = 0;
    int * check = nullptr;
};

#ifdef __CUDACC__
// A physical block id read from a block table: itself, or - in the bounds-checked build, when it is outside the
// pool - block 0 with the violation recorded (the kernel keeps its control flow and reads memory it owns).
__device__ __forceinline__ int rb_block(const KvLayout & kv, int blk) {
#ifdef RETRO_B200_CHECKED
    if (!rb_check_in_range(kv.check, CHECK_BLOCK, blk, kv.n_blocks)) return 0;
#endif
    return blk;
}
#endif

// `tile_tokens`: tokens per attention work item (a row of n tokens yields ceil(n / tile_tokens) items).
void launch_pack(const RowDesc * rows, int n_rows, int n_tokens, const int32_t * block_table, int max_blocks, int block_tokens,
                 int tile_tokens, PackMaps maps, cudaStream_t stream);
void launch_block_table_patch(int32_t * block_table, const int32_t * patches, int n_patches, cudaStream_t stream, int table_entries = 0, int n_blocks = 0,
                              int * check = nullptr);
void launch_kv_block_copy(KvLayout kv, int n_layer, const int32_t * pairs, int n_pairs, cudaStream_t stream);

// Sequence snapshots: dense is [layer][K|V][pos][head][row] for positions pos_first .. pos_first + n_pos - 1, a row
// being head_dim f16 values or the quantised pool's q_row_bytes.
void launch_kv_snapshot(KvLayout kv, int n_layer, const int32_t * table_row, int pos_first, int n_pos, void * dense, bool to_cache,
                        cudaStream_t stream);
// bytes of one (cell, head) row of the pool
inline int kv_row_bytes(int storage, int head_dim) {
    const int raw = storage == KV_Q8_0 ? head_dim + head_dim / 32 * 2 : storage == KV_Q4_0 ? head_dim / 2 + head_dim / 32 * 2 : head_dim * 2;
    return (raw + 7) & ~7;      // rows start on 8-byte boundaries
}
// Quantised pools. Store: the step's K (rotated) and V rows from the qkv buffer, quantised per 32 elements as ggml's
// quantize_row_q8_0_ref / quantize_row_q4_0_ref do. Dequant: every block that row r of the step may attend to
// (cu_rows / tok_* are the packing maps; `max_row_blocks` bounds the blocks of any row), into the f16 scratch; rows of
// at most `skip_tokens` tokens are left out (their attention kernel reads the pool itself); `n_scratch_rows` is the number
// of the other rows.
void launch_kv_quant_store(const float * qkv, int ld, int n_tokens, int n_head, KvLayout kv, int layer, const int32_t * tok_cell, cudaStream_t stream);
void launch_kv_dequant(KvLayout kv, int layer, int n_rows, int n_scratch_rows, int max_row_blocks, const int32_t * cu_rows, const int32_t * tok_slot,
                       const int32_t * tok_pos, const int32_t * tok_pos_min, int skip_tokens, cudaStream_t stream);

void launch_embed(WeightView embd, const int32_t * tokens, int n_tokens, float * x, cudaStream_t stream, int * check = nullptr);
// y[t] = x[gather ? gather[t] : t] * rsqrt(mean(x^2) + eps) * w
// `split`, when given (n a multiple of 32), also receives the row prepared for the tensor-core GEMM.
void launch_rms_norm(const float * x, int ldx, const int32_t * gather, const float * w, int n, float eps, float * y, int ldy, int n_tokens,
                     cudaStream_t stream, const SplitAct * split = nullptr);
// y[t][o] = sum_i deq(W)[o][i] x[t][i] (+ bias[o]) (+ residual[t][o]); reference kernel, any T.
void launch_gemm_rows(WeightView w, const float * x, int ldx, int n_tokens, float * y, int ldy, const float * bias, const float * residual,
                      int ldr, cudaStream_t stream);
// Exact variant (f32-grade accuracy): integer weight operand, two-term activation split.
bool gemm_q4k_exact_supported(const WeightView & w, const SplitAct & x);
void launch_gemm_q4k_exact(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                           const float * residual, int ldr, cudaStream_t stream);
// tcgen05 / tensor-memory variant of the exact GEMM (128 x 128 tiles). `error_flag` (device int) is
// raised if a pipeline wait inside the kernel timed out.
bool gemm_q4k_tc5_supported(const WeightView & w, const SplitAct & x);
// The grouped MXFP4 expert GEMM on tcgen05: rows [offsets[g], offsets[g + 1]) of x (the pairs sorted by expert) times
// expert g's bank (w.tiled, the tiled layout above; w.n_out rows per expert); y rows in the same order.
bool gemm_mxfp4_tc5_supported(const WeightView & w, const SplitAct & x);
void launch_gemm_mxfp4_tc5_grouped(const WeightView & w, int n_groups, const int32_t * group_offsets, const SplitAct & x, int total_rows, float * y,
                                   int ldy, int * error_flag, cudaStream_t stream);
// Whether the tcgen05 kernel's arithmetic covers these blocks (host memory, GGUF layout): it carries a row's
// minimum term as (dmin / d) * m inside the sum that d scales, so a super-block needs d != 0 unless its
// dmin * m are all zero, and |dmin / d * m| well inside the f16 range. Encoders produce nothing else.
bool q4k_min_fold_ok(const uint8_t * blocks, size_t n_blocks);
// With `scratch` (gemm_q4k_tc5_scratch_floats() floats) and few output tiles the reduction is cut into
// splits of whole super-blocks (grid.z) whose partial results a finish kernel adds in order.
int gemm_q4k_tc5_splits(uint32_t n_out, uint32_t n_in, int n_tokens, int n_sm);      // 1: the reduction is not split
size_t gemm_q4k_tc5_scratch_floats(uint32_t n_out, uint32_t n_in, int n_tokens, int n_sm);
void launch_gemm_q4k_tc5(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                         const float * residual, int ldr, int * error_flag, float * scratch, size_t scratch_floats, int n_sm, cudaStream_t stream,
                         const FinishTail * tail = nullptr);      // the tail is done only when the reduction is split
// Weight-streaming exact GEMM for at most 8 tokens. `scratch` holds gemm_q4k_stream_scratch_floats()
// floats of per-K-chunk partial sums; `n_sm` is the device's SM count (grid sizing); `error_flag` is set
// to 1 if a bounded wait on a copy gave up.
bool gemm_q4k_stream_supported(const WeightView & w, const SplitAct & x, int n_tokens);
size_t gemm_q4k_stream_scratch_floats(uint32_t n_out, uint32_t n_in);
void launch_gemm_q4k_stream(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                            const float * residual, int ldr, float * scratch, int n_sm, int * error_flag, cudaStream_t stream,
                            const FinishTail * tail = nullptr);
// y = sum over K chunks (in order) of partial sums laid out [chunk][t_stride tokens][n_out] + bias + residual,
// then the tail, if one is given and finish_tail_supported() (the caller checks).
void launch_gemm_stream_finish(const float * scratch, int n_chunks, int n_out, int n_tokens, int t_stride, float * y, int ldy, const float * bias,
                               const float * residual, int ldr, cudaStream_t stream, const FinishTail * tail = nullptr);
// Q8_0 counterpart of the streaming kernel. Its tile-major copy: one 2176-byte tile per (16 rows,
// 128 columns): the 16 x 4 block scales, then the int8 weights in MMA fragment order.
constexpr size_t kQ8TileBytes = 2176;
inline size_t q8_0_tiled_bytes(uint32_t n_out, uint32_t n_in) { return (size_t)((n_out + 15) / 16) * (n_in / 256) * 2 * kQ8TileBytes; }
void launch_q8_0_retile(const uint8_t * rows, uint32_t n_out, uint32_t n_in, uint32_t row_bytes, uint8_t * tiled, cudaStream_t stream);
bool gemm_q8_0_stream_supported(const WeightView & w, const SplitAct & x, int n_tokens);
void launch_gemm_q8_0_stream(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                             const float * residual, int ldr, float * scratch, int n_sm, int * error_flag, cudaStream_t stream,
                             const FinishTail * tail = nullptr);
// Q8_0 GEMM on tcgen05 for more than 16 tokens (weights as exact f16 pairs, three MMAs per product, one accumulator
// over the whole row); reads the GGUF-layout rows. q8_0_products_fit_f16 is the host-side check behind
// WeightView::tc5_exact for Q8_0 matrices. *error_flag is set to 1 if a bounded pipeline wait gave up.
bool q8_0_products_fit_f16(const uint8_t * blocks, size_t n_blocks);
bool gemm_q8_0_tc5_supported(const WeightView & w, const SplitAct & x);
void launch_gemm_q8_0_tc5(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias, const float * residual,
                          int ldr, int * error_flag, int n_sm, cudaStream_t stream);
// Exact tensor-core Q8_0 GEMM (mma.sync) for more than 8 tokens; reads the GGUF-layout rows.
bool gemm_q8_0_exact_supported(const WeightView & w, const SplitAct & x);
void launch_gemm_q8_0_exact(const WeightView & w, const SplitAct & x, int n_tokens, float * y, int ldy, const float * bias,
                            const float * residual, int ldr, cudaStream_t stream);
// Grouped form (expert banks): group g has its own matrix at w.data + g * group_stride_bytes (w describes one
// group's matrix) and the contiguous rows [group_offsets[g], group_offsets[g + 1]) of x and y (offsets on
// the device); max_group_rows bounds the largest group. One launch, 64-row token tiles whatever the
// group sizes, so a row's result does not depend on how the rows are grouped.
void launch_gemm_q8_0_exact_grouped(const WeightView & w, uint64_t group_stride_bytes, int n_groups, const int32_t * group_offsets, const SplitAct & x,
                                    int max_group_rows, float * y, int ldy, cudaStream_t stream);
// In-place RoPE on q and k (inside the fused qkv buffer) and the f16 store of k, v into the paged cache.
struct RopeStoreArgs {
    int n_head, n_head_kv, head_dim, n_rot;
    bool neox;
    const float * inv_freq;
    const int32_t * tok_pos;
    const int32_t * tok_cell;
    KvLayout kv;
    int layer;
};
// With `partial` the rows are first formed from a split-K GEMM's partial sums (laid out
// [chunk][t_stride tokens][ld_partial], added in chunk order, plus bias), each block its own columns.
void launch_rope_store(float * qkv, int ld, int n_tokens, const RopeStoreArgs & a, cudaStream_t stream, const float * partial = nullptr,
                       int n_chunks = 0, int t_stride = 0, int ld_partial = 0, const float * bias = nullptr);
bool rope_store_from_partial_supported(const RopeStoreArgs & a, const float * qkv, int ld, int n_out, const float * bias);
void launch_attention_ref(const float * qkv, int ld, int n_tokens, int n_head, KvLayout kv, int layer, const int32_t * tok_slot,
                          const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, cudaStream_t stream,
                          const SplitAct * split = nullptr);
// With `gather`: row t of the split form is row gather[t] / gather_div of x.
void launch_split_prep(const float * x, int ldx, int n, int n_tokens, const SplitAct & split, cudaStream_t stream, const int32_t * gather = nullptr,
                       int gather_div = 1);
// Tensor-core paged attention (head_dim 64 or 128, 16-token KV blocks, power-of-two GQA group). Work
// items hold at most kAttentionTileRows / G tokens.
constexpr int kAttentionTileRows = 128;
bool attention_mma_supported(int n_head, int n_head_kv, int head_dim, int block_tokens);
// `skip_small`: leave items of at most 16 query vectors to launch_attention_decode.
void launch_attention_mma(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items, const int32_t * tok_slot,
                          const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, bool skip_small, cudaStream_t stream);
// The same work on tcgen05 with TMA-staged K/V tiles: tensor maps over the K and V pools (all layers; boxes of
// one 16-token block x 64 columns, 128-byte swizzle), built once per engine. *error_flag is set to 1 if a bounded
// pipeline wait gave up.
struct AttentionMaps {
    CUtensorMap k, v;
    int valid = 0;
};
bool attention_maps_encode(AttentionMaps & maps, const __half * k, const __half * v, int head_dim, uint64_t rows);
bool attention_tc5_supported(int n_head, int n_head_kv, int head_dim, int block_tokens, const AttentionMaps & maps);
void launch_attention_tc5(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const AttentionMaps & maps, const int2 * items, int n_items,
                          const int32_t * tok_slot, const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, bool skip_small,
                          int * error_flag, cudaStream_t stream);
// Items of at most 16 query vectors (decode rows): the CTA's four warps split the KV blocks. Items of
// at most `min_cols` query vectors are left to launch_attention_decode8.
void launch_attention_decode(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items,
                             const int32_t * tok_slot, const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int min_cols,
                             cudaStream_t stream);
// Items of at most 8 query vectors, keys as the MMA's M dimension; `n_splits` CTAs share one item's KV
// blocks and a merge kernel combines them (`scratch`: attention_decode8_scratch_floats() floats). With
// more than one split and `split` given, the merge kernel also writes the output's split form (only
// complete when every row of the step belongs to such an item and head_dim % 32 == 0).
bool attention_decode8_supported(int n_head, int n_head_kv, int head_dim, int block_tokens);
int attention_decode8_max_splits();
size_t attention_decode8_scratch_floats(int n_items, int n_head_kv, int n_splits, int head_dim);
void launch_attention_decode8(const float * qkv, int ld, int n_head, KvLayout kv, int layer, const int2 * items, int n_items,
                              const int32_t * tok_slot, const int32_t * tok_pos, const int32_t * tok_pos_min, float * out, int ldo, int n_splits,
                              float * scratch, cudaStream_t stream, const SplitAct * split = nullptr);
// h[t][i] = silu(gu[t][i]) * gu[t][ff + i]
void launch_swiglu(const float * gu, int ld, int ff, int n_tokens, float * h, int ldh, cudaStream_t stream, const SplitAct * split = nullptr);

// MoE (CUDA-core kernels): router softmax + top-k, expert GEMMs grouped by expert, fixed-order combine.
void launch_moe_route(const float * router_logits, int n_expert, int k, int n_tokens, int32_t * ids, float * weights, cudaStream_t stream);
// The pairs of every expert in pair order (offsets[n_expert + 1], sorted[n_pairs]; n_expert <= 1024), and the
// grouped expert GEMM over them: an expert's rows are decoded once per eight of its pairs.
void launch_moe_group(const int32_t * pair_expert, int n_pairs, int n_expert, int32_t * offsets, int32_t * sorted, cudaStream_t stream);
void launch_moe_gemm_grouped(WeightView w_all, uint64_t expert_stride_bytes, int n_expert, const int32_t * offsets, const int32_t * sorted,
                             const float * x, int ldx, int x_div, float * y, int ldy, cudaStream_t stream);
void launch_moe_combine(const float * y_pairs, int ld, const int32_t * ids, const float * weights, int k, int d, int n_tokens,
                        const float * residual, float * out, cudaStream_t stream);

// Per-row LoRA (reference kernels): tmp[t][j] = A[a_t][j] . x[t]; y[t][o] += scale[a_t] * B[a_t][o] . tmp[t]
void launch_lora_shrink(const float * a_stack, int r_max, int n_in, const int32_t * tok_adapter, const float * x, int ldx, int n_tokens,
                        float * tmp, cudaStream_t stream);
// Segmented form of the shrink: tokens grouped by adapter with launch_moe_group(tok_adapter, n_tokens, n_adapters, ...);
// needs n_in % 4 == 0 and 16-byte aligned rows.
void launch_lora_shrink_grouped(const float * a_stack, int r_max, int n_in, int n_adapters, const int32_t * offsets, const int32_t * sorted,
                                const float * x, int ldx, float * tmp, cudaStream_t stream);
void launch_lora_expand(const float * b_stack, int r_max, int n_out, const float * scales, const int32_t * tok_adapter, const float * tmp,
                        int n_tokens, float * y, int ldy, cudaStream_t stream);

// Segmented LoRA on the tensor cores (TF32 MMAs on split operands, F32-accurate): shrink over K splits into
// tmp[target][split][t][r], then expand into y. Tokens grouped by
// adapter as for launch_lora_shrink_grouped.
constexpr int kLoraTcMaxSplits = 16;
int lora_tc_splits(int n_in);
bool lora_tc_supported(int r_max, int n_in, const float * a_stack, const float * x, int ldx);
// Up to three targets that read the same input rows: their A stacks [n_adapters][r_max][n_in], B stacks
// [n_adapters][n_out][r_max], widths and the column of y each one's result is added at. tmp holds
// kLoraTcMaxTargets * kLoraTcMaxSplits * n_tokens * r_max floats.
constexpr int kLoraTcMaxTargets = 3;
struct LoraGroup {
    const float * a[kLoraTcMaxTargets];
    const float * b[kLoraTcMaxTargets];
    int n_out[kLoraTcMaxTargets];
    int y_offset[kLoraTcMaxTargets];
    int n = 0;
};
void launch_lora_tc(const LoraGroup & group, const float * scales, int r_max, int n_in, int n_adapters, const int32_t * offsets, const int32_t * sorted,
                    const float * x, int ldx, int n_tokens, float * tmp, float * y, int ldy, cudaStream_t stream);

// Sampling over logits rows [S][n_vocab]. v2 rows transform their row of `work_logits`, which must
// then hold a copy of `raw_logits`; with v1 rows only, `work_logits` may be null.
// Rows whose flags carry bit 2 (v2, top_k == 1, no logit edits) are served by chunked arg-max kernels
// that need `scratch` (sample_scratch_bytes()); `n_greedy_fast` is how many rows carry the bit.
size_t sample_scratch_bytes(int n_vocab, int n_rows);
// `masks`: grammar rows carry in desc.pad[0] the word offset (plus one) of their one-bit-per-token mask; null without such rows.
void launch_sample(const float * raw_logits, float * work_logits, int n_vocab, int n_rows, const SampleDesc * desc, const LogitEdit * edits,
                   const uint32_t * masks, SampleOut * out, int32_t * top_ids, float * top_logprobs, int top_stride, int n_greedy_fast, void * scratch,
                   cudaStream_t stream);

} // namespace rb200
