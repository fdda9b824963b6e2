// Engine state behind the `retro_engine` handle: model weights in device memory, the paged KV
// cache with its block tables, per-request sampler state, per-row adapters and the step executor.
#pragma once

#include <functional>
#include <atomic>
#include <cstdlib>
#include "common.hpp"
#include "gguf.hpp"
#include "kernels.cuh"
#include "ep.hpp"
#include "kv.hpp"
#include "grammar.hpp"
#include "reasoning_budget.hpp"

#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/retro_b200.h"

// A grammar handle of the C ABI: an owned GBNF text (retro_grammar.cpp:1-76 in the reference).
struct retro_grammar {
    std::string gbnf;
};

namespace rb200 {

constexpr uint32_t kMaxSeq = 1024;        // sequence slots this backend accepts (the reference's fork caps at 256)
constexpr uint32_t kBlockTokens = 16;     // KV cells per block
constexpr int kStreamMaxTokens = 16;      // steps of at most this many tokens run the weight-streaming GEMMs (8 tokens per pass)

// Bumped whenever a device work buffer is (re)allocated; captured step graphs are dropped when it moves.
inline std::atomic<uint64_t> g_alloc_epoch{0};

template <class T> struct DeviceBuffer {
    T * ptr = nullptr;
    size_t count = 0;
    bool in_graphs = true;      // false for a temporary no captured step graph can hold: growing it leaves the graphs alone
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer & operator=(const DeviceBuffer &) = delete;
    ~DeviceBuffer() { if (ptr) cudaFree(ptr); }
    void ensure(size_t n) {
        if (n <= count) return;
        if (ptr) { cudaFree(ptr); ptr = nullptr; count = 0; }
        RB_CUDA(cudaMalloc(&ptr, n * sizeof(T)));
        count = n;
        if (in_graphs) ++g_alloc_epoch;        // captured CUDA graphs hold the old pointer
        // RB200_POISON=1 fills every new work buffer with 0xFF bytes (NaN as f32/f16): a read of
        // memory the step did not write then shows up in the results instead of depending on luck
        static const bool poison = std::getenv("RB200_POISON") != nullptr;
        if (poison) RB_CUDA(cudaMemset(ptr, 0xFF, n * sizeof(T)));
    }
};

// Kernel classes the optional per-step profile accumulates device time for.
enum KernelClass { K_GEMM = 0, K_ATTN, K_SAMPLE, K_PACK, K_MOE, K_LORA, K_OTHER, K_CLASS_COUNT };

// CUDA-event timing of kernel groups inside a step, on the stream the kernels are launched on.
// Off by default; when on, every group is bracketed by two events and the elapsed times are
// summed per class after the step's synchronisation.
struct StepProfiler {
    bool enabled = false;
    std::vector<cudaEvent_t> pool;
    size_t used = 0;
    struct Span { int cls; size_t e0, e1; uint32_t launches; };
    std::vector<Span> spans;
    double ms[K_CLASS_COUNT] = {};
    uint64_t launches[K_CLASS_COUNT] = {};
    size_t open_event = 0;
    ~StepProfiler() { for (cudaEvent_t e : pool) cudaEventDestroy(e); }
    size_t take() {
        if (used == pool.size()) {
            cudaEvent_t e;
            cudaEventCreate(&e);
            pool.push_back(e);
        }
        return used++;
    }
    void begin(int, cudaStream_t stream) {
        if (!enabled) return;
        open_event = take();
        cudaEventRecord(pool[open_event], stream);
    }
    void end(int cls, uint32_t n, cudaStream_t stream) {
        if (!enabled) return;
        const size_t e1 = take();
        cudaEventRecord(pool[e1], stream);
        spans.push_back({cls, open_event, e1, n});
    }
    void collect() {
        for (const Span & s : spans) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, pool[s.e0], pool[s.e1]) == cudaSuccess) {
                ms[s.cls] += t;
                launches[s.cls] += s.launches;
            }
        }
        spans.clear();
        used = 0;
    }
    void reset() {
        for (int i = 0; i < K_CLASS_COUNT; ++i) { ms[i] = 0; launches[i] = 0; }
    }
};

// Device storage of one SplitAct for up to `rows` rows of `ld` columns.
struct SplitBuffer {
    DeviceBuffer<__half> store;
    SplitAct view;
    void ensure(size_t rows, size_t ld) {
        if (ld % 32 != 0) return;
        const size_t main = rows * ld, sums = rows * (ld / 32);
        store.ensure(2 * main + 2 * sums + 64);
        view.hi = store.ptr;
        view.lo = store.ptr + main;
        view.sum_hi = store.ptr + 2 * main;
        view.sum_lo = store.ptr + 2 * main + sums + 32;
        view.ld = (int)ld;
        split_act_encode_maps(view, rows);
    }
    const SplitAct * get() const { return view.hi ? &view : nullptr; }
};

// MXFP4 blocks re-coded as Q8_0 blocks of the same values (see engine.cu); false when a block scale does not fit an f16.
bool mxfp4_to_q8_0(const void * src, size_t bytes, std::vector<uint8_t> & out);

struct HParams {
    std::string arch;
    uint32_t n_layer = 0, d = 0, n_head = 0, n_head_kv = 0, head_dim = 0, ff = 0, vocab = 0;
    uint32_t n_expert = 0, n_expert_used = 0, n_rot = 0;
    float eps = 1e-5f, rope_base = 10000.f;
    bool neox = false;
    uint32_t dq() const { return n_head * head_dim; }
    uint32_t dkv() const { return n_head_kv * head_dim; }
};

struct LayerWeights {
    const float * attn_norm = nullptr;
    WeightView wqkv;            // fused when the three projections share a storage type
    WeightView wq, wk, wv;      // otherwise
    const float * bqkv = nullptr;
    const float * q_norm = nullptr;
    const float * k_norm = nullptr;
    WeightView wo;
    const float * ffn_norm = nullptr;
    WeightView wgu;             // fused gate|up
    WeightView wgate, wup;
    WeightView wdown;
    // MoE
    WeightView router;          // F32 [n_expert][d]
    WeightView gate_exps, up_exps, down_exps;   // per-expert views (n_out = rows of one expert)
    uint64_t gate_stride = 0, up_stride = 0, down_stride = 0;
};

struct Model {
    HParams hp;
    WeightView token_embd;
    std::vector<LayerWeights> layers;
    const float * output_norm = nullptr;
    WeightView output;
    const float * output_bias = nullptr;
    DeviceBuffer<float> inv_freq;
    std::vector<void *> allocations;
    uint64_t weight_bytes = 0;
    uint64_t tiled_bytes = 0;
    std::vector<std::string> vocab_tokens;
    std::vector<int32_t> vocab_types;
    std::vector<retro_expert_bank_desc> expert_banks;   // as the GGUF holds them, sorted by tensor name
    std::vector<uint8_t> eog;                           // per token: ends a generation (EOS, EOT, EOM and the known end-of-turn pieces)
    bool is_eog(int32_t token) const { return token >= 0 && (size_t)token < eog.size() ? eog[token] != 0 : token == eos; }
    // The text of a token: byte-fallback pieces `<0xNN>` are one byte, U+2581 is a space, control pieces are empty
    // unless `unparse_special`.
    std::string piece(int32_t token, bool unparse_special) const;
    int32_t eos = 2, bos = 1;
    bool add_bos = true;
    ~Model() { for (void * p : allocations) cudaFree(p); }
};

struct Adapter {
    float scale = 1.f;
    uint32_t rank = 0;
    // target weight name -> (A [r][in], B [out][r]) in F32
    std::map<std::string, std::pair<std::vector<float>, std::vector<float>>> ab;
    uint64_t unpadded_bytes = 0;
    bool serial = false;        // registered by name for the one-active-at-a-time family, not selectable per row
};

// Monotonic prefix-reuse counters of the batched generators (retro_generation_stats).
struct GenerationCounters {
    uint64_t calls = 0, sequences = 0, prompt_tokens = 0, prefilled_tokens = 0, reused_tokens = 0, hits = 0, evictions = 0;
};

struct LoraTarget {
    DeviceBuffer<float> a;   // [n_adapters][r_max][n_in]
    DeviceBuffer<float> b;   // [n_adapters][n_out][r_max]
    uint32_t n_in = 0, n_out = 0;
    bool present = false;
};

struct RequestState {
    bool seeded = false;
    uint32_t seed = 0;
    uint64_t draws = 0;
    std::vector<int32_t> history;
    std::unique_ptr<GrammarState> grammar;      // v2 rows with a grammar: where the generation stands in it
    // reasoning budget: the plan the request's machine reads (a snapshot, the engine's may change under it), the
    // machine, and the end of the prompt collected across prefill chunks until the first sampling row primes it
    std::unique_ptr<ReasoningPlan> plan;
    BudgetMachine budget;
    bool primed = false;
    std::vector<int32_t> prompt_tail;
};

// A step row normalised from either ABI version.
struct EffRow {
    uint32_t struct_size;
    int32_t request, slot;
    const int32_t * tokens;
    uint32_t n;
    int32_t pos0;
    bool sample;
    retro_sampling_params v1;
    const retro_sampling_params_v2 * v2;
    uint32_t n_top_logprobs;
    bool want_logprob;
    int32_t adapter;
};

struct OutRow {
    int32_t token = 0;
    float logprob = 0.f;
    uint32_t n_top = 0;
    uint8_t forced = 0, sampled = 0;
    float sampled_logprob = 0.f;
};

class Engine {
public:
    Engine(const std::string & path, const retro_engine_config & config);
    ~Engine();

    int step(const EffRow * rows, size_t n_rows, OutRow * out, int32_t * top_ids, float * top_lps, size_t stride);
    int seq_rm(int32_t slot, int32_t p0, int32_t p1);
    int seq_cp(int32_t src, int32_t dst, int32_t p0, int32_t p1);
    int seq_pos(int32_t slot, int32_t * pmin, int32_t * pmax);
    int seq_save(int32_t slot, uint32_t flags, uint8_t * buffer, size_t n_buffer, size_t * out_n);
    int seq_load(int32_t slot, uint32_t flags, const uint8_t * buffer, size_t n_bytes, size_t * out_read);
    int memory(retro_engine_memory_info * out);
    int adapter_load(const char * path, float scale, int32_t * out_id);
    int adapter_unload(int32_t id);
    void adapter_info(retro_adapter_rows_info * out);
    // The one-active-at-a-time adapter family (rows with adapter == 0 decode under the active one).
    int lora_load_single(const char * path);
    int lora_load_named(const char * name, const char * path);
    int lora_activate(const char * name);
    int lora_set_enabled(bool enabled);
    const std::string & active_adapter() const { return active_name_; }
    int adapter_snapshot(int32_t replace, float scale, int32_t * out_id);
    void forget_kv();               // clears every slot and bumps the weights version
    uint64_t adapter_bytes() const;
    uint64_t work_buffer_bytes() const;
    GenerationCounters gen_stats;
    uint64_t route_pairs = 0;       // routed (token, expert) pairs served while telemetry was on
    int last_check[4] = {0, 0, 0, 0};       // bounds-checked build: the check word after the last step

    retro_engine_config config{};
    std::string model_path;
    uint64_t fingerprint = 0;
    uint64_t weights_version = 0;
    uint32_t n_ctx_seq = 0;
    std::unique_ptr<Model> model;
    std::unique_ptr<KvManager> kv;
    std::unordered_map<int32_t, RequestState> requests;
    // Reasoning budget (retro_engine_set_reasoning_budget): the tags as token ids from the caller's chat-template
    // layer, then the budget; -1 with the error set when the tags are unknown or outside the vocabulary.
    int set_reasoning_tags(const int32_t * start, size_t n_start, const int32_t * const * ends, const size_t * n_ends, size_t n_end_tags,
                           size_t n_prompt_tail);
    int set_reasoning_budget(int32_t budget);

    // inspection state of the last step
    size_t last_T = 0, last_S = 0, last_R = 0;
    float last_ms = 0.f;
    uint64_t last_launches = 0;
    // steps with more tokens than this take the tensor-core GEMM (f16 operands); fewer take the f32 row kernel
    int mma_min_tokens = 8;
    int tc5_min_tokens = 16;      // above this the tcgen05 kernel (128-token tiles) takes over; measured faster than mma.sync from 17 tokens on
    uint64_t last_h2d_bytes = 0, last_d2h_bytes = 0;
    StepProfiler prof_;
    uint64_t graphs_reused = 0;
    bool route_enabled = false;
    std::vector<std::vector<uint32_t>> route_counts;   // [layer][expert]

    // device state exposed to the inspection entry points
    PackMaps maps{};
    DeviceBuffer<float> logits;
    DeviceBuffer<int32_t> route_ids;     // [layer][T][k]
    cudaStream_t stream = nullptr;
    const int32_t * kv_block_table_device() const { return block_table_.ptr; }

    // Expert parallelism (MoE models): joins an NCCL communicator of `world` engines, one per GPU;
    // from then on every MoE layer exchanges its (token, expert) pairs with the experts' ranks, and
    // all ranks must run the same number of steps (a rank without rows calls ep_idle_step()).
    void ep_init(int rank, int world, const void * unique_id_128);
    void ep_idle_step();
    void ep_keep_local_experts();
    size_t ep_local_bank_bytes_ = 0;     // bytes of expert banks this rank holds once it joined an expert-parallel group
    int ep_world() const { return ep_world_; }

private:
    void load_model(const std::string & path);
    void restack_adapters();
    bool moe_experts_on_tensor_cores(const LayerWeights & lw) const;
    void moe_experts_tc(const LayerWeights & lw, const float * rows, int ld_rows, const int32_t * gather, int gather_div, const int32_t * d_offsets,
                        int n, float * y_out, int ld_out);
    void ep_moe_layer(const LayerWeights & lw, int T);
    bool ep_agree(bool ready);
    void ep_exchange(const float * send, const std::vector<int32_t> & send_begin, const std::vector<int32_t> & send_count, float * recv,
                     const std::vector<int32_t> & recv_begin, const std::vector<int32_t> & recv_count, int d);
    bool tc5_split_preferred(const WeightView & w, int T, const SplitAct * xs) const;
    bool linear(const WeightView & w, const float * x, int ldx, int T, float * y, int ldy, const float * bias, const float * residual, int ldr,
                const SplitAct * xs = nullptr, const FinishTail * tail = nullptr);
    struct GraphEntry {
        std::vector<uint64_t> sig;
        cudaGraphExec_t exec = nullptr;
        uint32_t launches = 0;
        int seen = 0;
        bool failed = false;
    };
    std::unordered_map<uint64_t, GraphEntry> graphs_;
    uint64_t graph_epoch_ = 0;
    uint64_t graph_replays_ = 0;
    bool graphs_enabled_ = true;
    void run_step_work(const std::vector<uint64_t> & sig, const std::function<void()> & issue);
  public:
    void graph_stats(uint64_t * replays, uint64_t * cached) const { if (replays) *replays = graph_replays_; if (cached) *cached = graphs_.size(); }
  private:
    bool linear_reads_split(const WeightView & w, int ldx, int T, const SplitAct * xs) const;
    void lora(const std::string & target, const float * x, int ldx, int T, float * y, int ldy);
    void lora_group(const std::vector<std::string> & targets, const std::vector<int> & y_offsets, const float * x, int ldx, int T, float * y, int ldy);
    void flush_kv_updates();
    KvLayout kv_layout() const;

    DeviceBuffer<__half> kcache_, vcache_;             // the F16 pool (every layer), or - over a quantised pool - one layer of f16 scratch
    uint64_t kv_layer_stride_ = 0;
    DeviceBuffer<uint8_t> kq_, vq_;                    // the quantised pool (kv_dtype Q8_0 / Q4_0)
    uint64_t kv_q_layer_stride_ = 0;                   // bytes per layer
    int32_t kv_storage_ = KV_F16;
    bool kv_q8_native_ = true;                         // decode rows read a quantised pool directly (RB200_KV_Q8_NATIVE=0: through the scratch)
    DeviceBuffer<int32_t> block_table_;
    DeviceBuffer<int32_t> maps_store_;
    DeviceBuffer<uint8_t> d_stage_;
    uint8_t * h_stage_ = nullptr;
    size_t stage_bytes_ = 0;
    DeviceBuffer<uint8_t> d_result_;
    uint8_t * h_result_ = nullptr;
    size_t result_bytes_ = 0;
    DeviceBuffer<float> x_, xn_, qkv_, att_, gu_, hff_, hs_, router_logits_, moe_w_, pair_gu_, pair_h_, pair_y_, lora_tmp_, logits_work_;
    DeviceBuffer<int32_t> moe_ids_, d_aux_;
    DeviceBuffer<int32_t> moe_offsets_, moe_sorted_, lora_offsets_, lora_sorted_;
    DeviceBuffer<int> device_error_;
    DeviceBuffer<int> check_word_;      // bounds-checked build: {code, value, limit, count} of the first violation
    DeviceBuffer<float> stream_scratch_;
    DeviceBuffer<uint8_t> sample_scratch_;
    DeviceBuffer<float> attn_scratch_;
    bool attn_decode8_ = true;
    int n_sm_ = 148;
    bool stream_gemm_ = true;
    bool moe_tensor_cores_ = true;      // RB200_MOE=rows: experts stay MXFP4 on the CUDA-core row kernel
    bool q8_tc5_ = true;                // RB200_Q8_TC5=0: Q8_0 above 16 tokens stays on the mma.sync kernel
    bool lora_tensor_cores_ = true;     // RB200_LORA=rows: the CUDA-core shrink / expand kernels instead
    DeviceBuffer<float> moe_xs_, moe_gu_s_, moe_y_s_;      // expert-contiguous rows: inputs, [gate | up], outputs
    SplitBuffer moe_x_split_, moe_h_split_;
    size_t moe_split_rows_ = 0;
    void * ep_comm_ = nullptr;
    int ep_rank_ = 0, ep_world_ = 1;
    EpPlan ep_plan_;
    int32_t * h_ep_offsets_ = nullptr;        // pinned: every rank's pair offsets of the layer
    DeviceBuffer<int32_t> ep_all_offsets_, ep_offsets_l_, ep_sorted_l_, ep_flags_;
    DeviceBuffer<float> ep_send_, ep_recv_, ep_gu_, ep_h_, ep_y_, ep_back_;
    bool fused_finish_ = true;      // RB200_FUSED_FINISH=0: norm / SwiGLU always as kernels of their own
    SplitBuffer xn_split_, att_split_, hff_split_, hs_split_;
    cudaEvent_t ev_begin_ = nullptr, ev_end_ = nullptr;
    cudaStream_t side_stream_ = nullptr;                 // decode-row attention beside the prefill tiles
    cudaEvent_t ev_fork_ = nullptr, ev_join_ = nullptr;
    bool attn_overlap_ = true;                           // RB200_ATTN_OVERLAP=0: every attention kernel on the step's stream

    bool read_adapter_file(const char * path, float scale, Adapter & out);
    std::map<std::string, int32_t> serial_ids_;      // name -> id in adapters_
    std::string active_name_;
    int32_t active_id_ = 0;
    ReasoningPlan reasoning_plan_;                  // active when tags and a budget >= 0 are set
    bool reasoning_seen_ = false;                   // some request may still hold a machine
    std::vector<std::string> token_pieces_;         // every token's text, built when the first grammar row arrives
    std::map<int32_t, Adapter> adapters_;
    std::map<int32_t, int32_t> adapter_index_;   // id -> stack index
    int32_t next_adapter_id_ = 1;
    uint32_t r_max_ = 0;
    std::map<std::string, std::unique_ptr<LoraTarget>> lora_targets_;
    DeviceBuffer<float> lora_scales_;
    uint64_t stacked_bytes_ = 0;
    const int32_t * cur_tok_adapter_ = nullptr;
    bool cur_any_adapter_ = false;
    bool attn_mma_ = false;
    bool attn_tc5_ = false;             // prefill tiles on the tcgen05 kernel (needs the K/V tensor maps)
    AttentionMaps attn_maps_;
    int attn_tile_tokens_ = 64;
};

} // namespace rb200
