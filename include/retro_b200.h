/* C ABI of libretro_b200: the batched decode step of the step-wise generation engine,
 * implemented with CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * Every `retro_engine_*` / `retro_last_error` declaration below replaces the entry point of the
 * same name in the reference's runtime header
 * crates/retrograd-ffi/runtime/include/retro_lora_train.h (line ranges cited per group); struct
 * layouts are byte-identical to it (checked by static_asserts in the implementation, mirroring
 * crates/retrograd-ffi/src/lib.rs:2825-3060). Status codes: 0 ok, -1 runtime error, -2 buffer
 * too small, -3 invalid argument (reported before anything is decoded); constructors return
 * NULL. The message of the last failure on the calling thread is read with retro_last_error().
 *
 * `retro_b200_*` entry points have no counterpart in the reference: they are the inspection
 * hooks the parity tests and the benchmark need (packing maps, block tables, logits, timing,
 * model synthesis).
 */
#ifndef RETRO_B200_H
#define RETRO_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* retro_lora_train.h:3038 */
const char * retro_last_error(void);

/* ---- shared value types (retro_lora_train.h:1229-1242,1255-1393,1472-1482) ---- */

typedef struct retro_sampling_params {
    float    temperature;
    float    top_p;
    uint32_t max_new_tokens;
    uint32_t seed;
} retro_sampling_params;

#define RETRO_STATE_SEQ_FLAGS_NONE         0u
#define RETRO_STATE_SEQ_FLAGS_PARTIAL_ONLY 1u
#define RETRO_STATE_SEQ_FLAGS_ON_DEVICE    2u

#define RETRO_STEP_ADAPTER_BASE (-1)

typedef struct retro_step_row {
    uint32_t struct_size;
    int32_t  request;
    int32_t  slot;
    const int32_t * tokens;
    uint32_t n;
    int32_t  pos0;
    bool     sample;
    retro_sampling_params sampling;
    uint32_t n_top_logprobs;
    int32_t  adapter;
} retro_step_row;

typedef struct retro_adapter_rows_info {
    uint32_t struct_size;
    uint32_t n_adapters;
    uint32_t max_rank;
    uint64_t stacked_bytes;
    uint64_t unpadded_bytes;
} retro_adapter_rows_info;

typedef struct retro_step_out_row {
    uint32_t struct_size;
    int32_t  token;
    float    logprob;
    uint32_t n_top;
    uint8_t  forced;
    uint8_t  sampled;
} retro_step_out_row;

typedef struct retro_grammar retro_grammar;

typedef struct retro_sampling_params_v2 {
    uint32_t struct_size;
    float    temperature;
    float    top_p;
    uint32_t max_new_tokens;
    uint32_t seed;
    int32_t  top_k;
    float    min_p;
    float    repeat_penalty;
    float    frequency_penalty;
    float    presence_penalty;
    uint32_t penalty_window;
    uint32_t n_logit_bias;
    const int32_t * logit_bias_ids;
    const float   * logit_bias_values;
    const retro_grammar * grammar;
} retro_sampling_params_v2;

typedef struct retro_step_row_v2 {
    uint32_t struct_size;
    int32_t  request;
    int32_t  slot;
    const int32_t * tokens;
    uint32_t n;
    int32_t  pos0;
    bool     sample;
    retro_sampling_params_v2 sampling;
    uint32_t n_top_logprobs;
    uint8_t  want_logprob;
    int32_t  adapter;
} retro_step_row_v2;

typedef struct retro_step_out_row_v2 {
    uint32_t struct_size;
    int32_t  token;
    float    logprob;
    uint32_t n_top;
    uint8_t  forced;
    uint8_t  sampled;
    float    sampled_logprob;
} retro_step_out_row_v2;

typedef struct retro_engine_memory_info {
    uint32_t struct_size;
    uint32_t n_slots;
    uint64_t cells_total;
    uint64_t cells_used;
    uint64_t kv_bytes;
    uint64_t recurrent_bytes;
} retro_engine_memory_info;

/* ---- engine handle (retro_lora_train.h:2465-2509) ---- */

typedef struct retro_engine retro_engine;
typedef struct retro_trainer retro_trainer;   /* the trainer handle of the trainer-owned generation context (below) */

enum retro_engine_kv_dtype {
    RETRO_ENGINE_KV_DTYPE_F32 = 0,
    RETRO_ENGINE_KV_DTYPE_F16 = 1,
    RETRO_ENGINE_KV_DTYPE_Q8_0 = 2,
    RETRO_ENGINE_KV_DTYPE_Q4_0 = 3,
};

enum retro_device {
    RETRO_DEVICE_AUTO = 0,
    RETRO_DEVICE_CPU = 1,
    RETRO_DEVICE_GPU = 2,
};

enum retro_expert_placement {
    RETRO_EXPERT_PLACEMENT_DEVICE = 0,
    RETRO_EXPERT_PLACEMENT_HOST = 1,
};

typedef struct retro_engine_config {
    uint32_t struct_size;
    uint32_t n_ctx;
    uint32_t n_seq_max;
    uint32_t n_batch;
    uint32_t n_ubatch;
    int32_t  kv_dtype;
    bool     flash_attn;
    int32_t  device;
    uint32_t threads;
    bool     verbose;
    uint32_t kv_unified;
    int32_t  expert_placement;
    uint32_t expert_host_layers;
    uint64_t expert_device_cache_bytes;
} retro_engine_config;

retro_engine * retro_engine_new(const char * model_path, const retro_engine_config * config);
retro_engine * retro_engine_new_checked(const char * model_path, const retro_engine_config * config,
                                        bool * out_invalid_placement);
void retro_engine_free(retro_engine * engine);

/* ---- vocabulary introspection (retro_lora_train.h:2538-2561) ---- */
int retro_engine_eos_token(retro_engine * engine, int32_t * out_token);
int retro_engine_vocab_size(retro_engine * engine, uint32_t * out_n_vocab);
int retro_engine_is_eog_token(retro_engine * engine, int32_t token, bool * out_is_eog);

/* Reasoning budget (reference: retro_engine_set_reasoning_budget, retro_lora_train.h:2622-2627, and the trainer's
 * retro_trainer_set_reasoning_budget, :1680-1688): -1 lets the model decide, N >= 0 forces the reasoning block's
 * end tag after N reasoning tokens; rows report forced tokens in `forced`. Each request carries its own machine,
 * primed from the end of its prompt (retro_gen_core.cpp:890-1007, 2609-2680). The reference reads the tags out of
 * the model's chat template; this library renders no templates: the caller's template layer passes them as token
 * ids with retro_b200_engine_set_reasoning_tags first, and a budget >= 0 without tags fails with the reference's
 * message for a template that declares no reasoning block. -1 on refusal, with the error set. */
int retro_engine_set_reasoning_budget(retro_engine * engine, int32_t budget);
int retro_trainer_set_reasoning_budget(retro_trainer * trainer, int32_t budget);
/* No counterpart in the reference (there the tags come from common_chat_templates_apply,
 * retro_chat_parser.cpp:558-640): the opening tag, the closing tags (the first one is the tag a spent budget
 * forces) and the number of prompt tokens at the end of a prompt that are replayed into a fresh machine (the
 * length of the template's generation prompt). */
int retro_b200_engine_set_reasoning_tags(retro_engine * engine, const int32_t * start, size_t n_start, const int32_t * const * end_tags,
                                         const size_t * n_end, size_t n_end_tags, size_t n_prompt_tail);
int retro_b200_trainer_set_reasoning_tags(retro_trainer * trainer, const int32_t * start, size_t n_start, const int32_t * const * end_tags,
                                          const size_t * n_end, size_t n_end_tags, size_t n_prompt_tail);
/* Host logic only (no GPU): one request's budget machine, primed with the end of `prompt` and then fed the tokens
 * a sampler drew; out_tokens[i] is what the step would emit in place of sampled[i], out_forced[i] whether the
 * budget forced it. `incomplete` lists token ids whose text stops inside a UTF-8 sequence. */
int retro_b200_reasoning_check(const int32_t * start, size_t n_start, const int32_t * const * end_tags, const size_t * n_end, size_t n_end_tags,
                               int32_t budget, size_t n_prompt_tail, const int32_t * prompt, size_t n_prompt, const int32_t * incomplete,
                               size_t n_incomplete, const int32_t * sampled, size_t n_sampled, int32_t * out_tokens, uint8_t * out_forced);
int retro_engine_context_size(retro_engine * engine, uint32_t * out_n_ctx);
int retro_engine_detokenize(retro_engine * engine, const int32_t * tokens, size_t n_tokens, bool unparse_special,
                            char * buffer, size_t n_buffer, size_t * out_n_bytes);
int retro_engine_tokenize_text(retro_engine * engine, const char * text, int32_t * tokens, size_t n_tokens_max,
                               size_t * out_n_tokens);
int retro_engine_tokenize_fragment(retro_engine * engine, const char * text, int32_t * tokens, size_t n_tokens_max,
                                   size_t * out_n_tokens);

/* ---- per-row adapters (retro_lora_train.h:2597-2612) ---- */
int retro_engine_adapter_load(retro_engine * engine, const char * adapter_path, float scale, int32_t * out_id);
int retro_engine_adapter_unload(retro_engine * engine, int32_t id);
int retro_engine_adapter_rows_info(retro_engine * engine, retro_adapter_rows_info * out_info);
int retro_engine_graphs_reused(retro_engine * engine, uint64_t * out_n_reused);

/* ---- step-wise generation (retro_lora_train.h:2712-2719,1410-1417) ---- */
int retro_engine_step(retro_engine * engine, const retro_step_row * rows, size_t n_rows, retro_step_out_row * out_rows,
                      int32_t * out_top_ids, float * out_top_logprobs, size_t n_top_stride);
int retro_engine_step_v2(retro_engine * engine, const retro_step_row_v2 * rows, size_t n_rows,
                         retro_step_out_row_v2 * out_rows, int32_t * out_top_ids, float * out_top_logprobs,
                         size_t n_top_stride);

/* ---- sequence memory (retro_lora_train.h:2721-2775) ---- */
int retro_engine_seq_rm(retro_engine * engine, int32_t slot, int32_t p0, int32_t p1);
int retro_engine_seq_cp(retro_engine * engine, int32_t src, int32_t dst, int32_t p0, int32_t p1);
int retro_engine_seq_save(retro_engine * engine, int32_t slot, uint32_t flags, uint8_t * buffer, size_t n_buffer,
                          size_t * out_n_bytes);
int retro_engine_seq_load(retro_engine * engine, int32_t slot, uint32_t flags, const uint8_t * buffer, size_t n_bytes,
                          size_t * out_n_read);
int retro_engine_seq_pos(retro_engine * engine, int32_t slot, int32_t * out_pos_min, int32_t * out_pos_max);
int retro_engine_memory(retro_engine * engine, retro_engine_memory_info * out);
/* Batched generators over the step path (retro_lora_train.h:1238-1242, 1845-1880, 2511-2534;
 * retro_gen_core.cpp:1696-1877, 1878-2049). Outputs are row-major with a stride of n_out_max; a row
 * stops at max_new_tokens, at an end-of-generation token (included), at n_out_max or when its
 * context fills. out_logprobs (temperature-1 policy logprobs) and out_forced (always 0 here) may be
 * NULL. Both calls forget every resident sequence before and after, as the reference does without
 * its generation prefix cache. Sampling runs on the GPU: greedy-equivalent settings are exact, seeded
 * rows follow this library's counter-based generator. */
typedef struct retro_generation_sequence {
    const int32_t * prompt_tokens;
    size_t n_prompt;
    retro_sampling_params sampling;
} retro_generation_sequence;
/* One prompt, n_sequences samples: the prompt is decoded once, its memory shared with every member. */
int retro_engine_generate_batch(retro_engine * engine, const int32_t * prompt_tokens, size_t n_prompt, const retro_sampling_params * sampling,
                                size_t n_sequences, int32_t * out_tokens, float * out_logprobs, size_t n_out_max, size_t * out_n_tokens,
                                uint8_t * out_forced);
/* One completion per (prompt, sampling) pair. */
int retro_engine_generate_continuous_batch(retro_engine * engine, const retro_generation_sequence * sequences, size_t n_sequences,
                                           int32_t * out_tokens, float * out_logprobs, size_t n_out_max, size_t * out_n_tokens,
                                           uint8_t * out_forced);

int retro_engine_request_free(retro_engine * engine, int32_t request);
int retro_engine_kv_unified(retro_engine * engine, bool * out_unified);

/* ---- cache keys (retro_lora_train.h:2796-2808) ---- */
int retro_engine_weights_version(retro_engine * engine, uint64_t * out_version);
int retro_engine_model_fingerprint(retro_engine * engine, uint64_t * out_fingerprint);
int retro_engine_is_hybrid(retro_engine * engine, bool * out_is_hybrid);

/* ---- MoE routing telemetry (retro_lora_train.h:2791-2794) ---- */
int retro_engine_expert_route_enable(retro_engine * engine, uint32_t sample_every);
int retro_engine_expert_route_counts(retro_engine * engine, uint32_t layer, uint32_t * out, size_t n_expert);
int retro_engine_expert_route_reset(retro_engine * engine);

/* ---- serialised adapters: one active at a time (retro_lora_train.h:2566-2584, 2616-2620) ----
 * Rows of a step whose `adapter` is 0 decode under the active adapter (the base model when none is
 * active). load_lora replaces every registered adapter and activates the file; load_lora_named
 * registers a file beside the others and re-applies it only when it is the active one; activate_lora
 * (NULL or "" = the base model) and set_lora_enabled switch. Every activation, enable or disable
 * clears the whole KV and bumps the weights version (retro_engine.cpp:322-328). */
int retro_engine_load_lora(retro_engine * engine, const char * adapter_path);
int retro_engine_set_lora_enabled(retro_engine * engine, bool enabled);
int retro_engine_load_lora_named(retro_engine * engine, const char * name, const char * adapter_path);
int retro_engine_activate_lora(retro_engine * engine, const char * name);
/* The active adapter's name (empty: the base model). Two-call string contract: with buffer NULL or
 * n_buffer 0 only *out_n_bytes is written; otherwise the text plus a NUL, -2 when it does not fit. */
int retro_engine_active_adapter(retro_engine * engine, char * buffer, size_t n_buffer, size_t * out_n_bytes);

/* ---- counters and memory (retro_lora_train.h:849-917, 1113-1131, 2666-2674) ---- */
typedef struct retro_memory_report {
    uint64_t model_weight_bytes;
    uint64_t optimizer_kv_bytes;
    uint64_t optimizer_compute_bytes;
    uint64_t generation_kv_bytes;
    uint64_t generation_compute_bytes;
    bool     has_generation_context;
    uint64_t trainable_parameter_bytes;
    uint64_t trainable_gradient_bytes;
    uint64_t optimizer_state_bytes;
    bool     trainable_parameters_are_model_subset;
    bool     adapter_on_host;
    bool     base_trainable_on_host;
    uint64_t device_bytes;
    uint64_t host_bytes;
    uint64_t device_total_bytes;
    uint64_t device_used_bytes;
    uint64_t device_peak_used_bytes;
    uint64_t backend_scratch_bytes;
    uint64_t backend_scratch_peak_bytes;
    uint64_t device_memory_samples;
    uint64_t checkpoint_count;
    uint64_t checkpoint_retained_bytes;
    uint64_t checkpoint_live_peak_bytes;
    uint64_t checkpoint_live_peak_count;
    uint64_t checkpoint_long_lived_bytes;
    uint64_t checkpoint_long_lived_count;
    uint64_t checkpoint_graph_nodes;
    uint64_t checkpoint_max_span_nodes;
    uint64_t checkpoint_total_span_nodes;
} retro_memory_report;
/* Weights (both layouts of a quantised matrix count), KV pool, work buffers, adapters (their bytes
 * are `trainable_parameter_bytes`, as the reference reports an engine's adapters), everything on the
 * device; optimizer, gradient and checkpoint fields are zero: the handle has none. The measured fields
 * come from one cudaMemGetInfo sample. */
int retro_engine_memory_report(retro_engine * engine, retro_memory_report * out_report);

typedef struct retro_generation_stats {
    uint64_t calls;
    uint64_t sequences;
    uint64_t prompt_tokens;
    uint64_t prefilled_tokens;
    uint64_t reused_tokens;
    uint64_t hits;
    uint64_t evictions;
} retro_generation_stats;
/* Monotonic prefix-reuse counters of the batched generators: a shared prompt decoded once and
 * attached to n - 1 more sequences counts n - 1 hits and (n - 1) * (n_prompt - 1) reused tokens. */
int retro_engine_generation_stats(retro_engine * engine, retro_generation_stats * out_stats);

/* ---- MoE expert banks (retro_lora_train.h:742-758, 788-795, 827-840, 2780-2793) ---- */
#define RETRO_MODEL_INFO_NAME_MAX 64
#define RETRO_TENSOR_NAME_MAX 128
typedef struct retro_tensor_desc {
    char name[RETRO_TENSOR_NAME_MAX];
    int64_t ne[4];
    uint64_t n_elements;
    uint64_t n_bytes;
    uint64_t storage_id;
    char type_name[RETRO_MODEL_INFO_NAME_MAX];
} retro_tensor_desc;
typedef struct retro_expert_bank_desc {
    uint32_t layer;
    char role[16];
    retro_tensor_desc tensor;
} retro_expert_bank_desc;
#define RETRO_EXPERT_CACHE_MAX_GROUPS 16
typedef struct retro_expert_cache_group {
    int32_t  n_slots;
    int32_t  n_layers;
    int32_t  n_expert;
    uint64_t device_bytes;
} retro_expert_cache_group;
typedef struct retro_expert_cache_stats {
    struct { uint64_t hits; uint64_t misses; uint64_t bytes; } small;
    struct { uint64_t hits; uint64_t misses; uint64_t bytes; } large;
    struct { uint64_t hits; uint64_t misses; uint64_t bytes; } copy;
    int32_t n_groups;
    retro_expert_cache_group groups[RETRO_EXPERT_CACHE_MAX_GROUPS];
} retro_expert_cache_stats;
/* The `ffn_{gate,up,down}_exps` banks of the loaded model as the GGUF holds them (name, shape, bytes,
 * type), sorted by tensor name. Two-call contract: out_banks NULL and n_max 0 report the count; a short
 * buffer fails with -2. */
int retro_engine_expert_banks(retro_engine * engine, retro_expert_bank_desc * out_banks, size_t n_max, size_t * out_count);
/* Counters of the expert device cache: every bank is resident on the device here, so there is no
 * cache and the struct is zeroed. */
int retro_engine_expert_stats(retro_engine * engine, retro_expert_cache_stats * out_stats);
/* How routed (token, expert) pairs were served since telemetry was enabled: out[0] from resident
 * device banks (all of them here), out[1] by a copy, out[2] by a read-back (always 0). */
int retro_engine_expert_route_paths(retro_engine * engine, uint64_t out[3]);

/* ---- grammar handles (retro_lora_train.h:1395-1408): host-only owners of a GBNF text ---- */
/* from_json_schema returns NULL with a message: the schema converter is part of the reference's
 * llama.cpp fork and is not restated here; pass GBNF. The handle may be freed as soon as the step
 * call that carried it returns. */
retro_grammar * retro_grammar_from_json_schema(const char * json_schema);
retro_grammar * retro_grammar_from_gbnf(const char * gbnf);
retro_grammar * retro_grammar_json_object(void);
const char *    retro_grammar_gbnf(const retro_grammar * grammar);
void            retro_grammar_free(retro_grammar * grammar);

/* ---- the trainer-owned generation context (retro_lora_train.h:1410-1417 twin, 1427-1455, 1906-1945) ----
 * The reference's RL trainer drives the same step path on its own generation context through
 * retro_trainer_generation_*: same structs, same contracts as the engine entry points. The training
 * runtime behind `retro_trainer` is not part of this library; a handle made by
 * retro_b200_trainer_generation_new (below) owns only that generation context, and the host calls
 * retro_b200_trainer_weights_updated after each optimizer step or weight import, which does what the
 * reference's forget_generation_kv() does there: clears the KV and bumps the weights version so every
 * prefix cache keyed on it drops its entries (crates/retrograd-infer/src/scheduler.rs:548-560). */
typedef struct retro_trainer retro_trainer;
int retro_trainer_generation_step(retro_trainer * trainer, const retro_step_row * rows, size_t n_rows, retro_step_out_row * out_rows,
                                  int32_t * out_top_ids, float * out_top_logprobs, size_t n_top_stride);
int retro_trainer_generation_step_v2(retro_trainer * trainer, const retro_step_row_v2 * rows, size_t n_rows,
                                     retro_step_out_row_v2 * out_rows, int32_t * out_top_ids, float * out_top_logprobs,
                                     size_t n_top_stride);
int retro_trainer_generation_seq_rm(retro_trainer * trainer, int32_t slot, int32_t p0, int32_t p1);
int retro_trainer_generation_seq_cp(retro_trainer * trainer, int32_t src, int32_t dst, int32_t p0, int32_t p1);
int retro_trainer_generation_seq_save(retro_trainer * trainer, int32_t slot, uint32_t flags, uint8_t * buffer, size_t n_buffer,
                                      size_t * out_n_bytes);
int retro_trainer_generation_seq_load(retro_trainer * trainer, int32_t slot, uint32_t flags, const uint8_t * buffer, size_t n_bytes,
                                      size_t * out_n_read);
int retro_trainer_generation_seq_pos(retro_trainer * trainer, int32_t slot, int32_t * out_pos_min, int32_t * out_pos_max);
int retro_trainer_generation_memory(retro_trainer * trainer, retro_engine_memory_info * out);
int retro_trainer_generation_request_free(retro_trainer * trainer, int32_t request);
int retro_trainer_generation_kv_unified(retro_trainer * trainer, bool * out_unified);
int retro_trainer_generation_weights_version(retro_trainer * trainer, uint64_t * out_version);
int retro_trainer_generation_stats(retro_trainer * trainer, retro_generation_stats * out_stats);
/* A frozen copy of the trained (= active) adapter as a per-row adapter; `replace`, when not 0, is
 * unloaded first. Refused when no adapter is active. */
int retro_trainer_generation_adapter_snapshot(retro_trainer * trainer, int32_t replace, float scale, int32_t * out_id);
int retro_trainer_generation_adapter_unload(retro_trainer * trainer, int32_t id);
int retro_trainer_generation_adapter_rows_info(retro_trainer * trainer, retro_adapter_rows_info * out_info);

/* ================= extensions without a counterpart in the reference ================= */

/* Host-only check of a text against a GBNF grammar with the engine the step path uses for grammar rows:
 * *out_state = 0 the text is rejected, 1 it is a valid prefix, 2 it matches the root rule completely; -3 and the
 * parser's message for an invalid grammar. */
int retro_b200_grammar_check(const char * gbnf, const char * text, int * out_state);

/* The bounds-checked build (libretro_b200_checked.so, compiled with -DRETRO_B200_CHECKED): every index a kernel
 * reads from device memory (token ids, slots, positions, block-table entries, block ids, adapter indices) is
 * compared with its range before use; a violation skips the access, is recorded, and makes the step return -1
 * with the value and its range in the message. retro_b200_checked_build() tells which build is loaded (1 / 0);
 * retro_b200_engine_check_word() returns {code, value, limit, violations} of the last step (all zero in the
 * normal build and after a clean step). */
int retro_b200_checked_build(void);
int retro_b200_engine_check_word(retro_engine * engine, int32_t out_word_4[4]);

/* A `retro_trainer` that owns nothing but a generation context (see the retro_trainer_generation_*
 * group above); `adapter_path`, when not NULL, is the trained adapter the context decodes under.
 * retro_b200_trainer_weights_updated is the host's notice that the weights behind the context changed. */
retro_trainer * retro_b200_trainer_generation_new(const char * model_path, const retro_engine_config * config, const char * adapter_path);
void retro_b200_trainer_generation_free(retro_trainer * trainer);
int retro_b200_trainer_weights_updated(retro_trainer * trainer, const char * adapter_path);


/* Writes a seeded random model as GGUF. `spec` is whitespace-separated key=value pairs:
 * arch(llama|qwen2|olmoe) layers d heads kv_heads head_dim ff vocab experts experts_used
 * dtype expert_dtype embd_dtype (f32|f16|q8_0|q4_k|mxfp4) std seed bias rope_base eps dist eot turn_end
 * (eot: a token id named by tokenizer.ggml.eot_token_id; turn_end: a token id only spelled as an end-of-turn piece). */
int retro_b200_synth_gguf(const char * path, const char * spec, uint64_t * out_bytes);

/* Encodes `n` floats as one stored row of `ggml_type` (0 f32, 1 f16, 8 q8_0, 12 q4_K, 39 mxfp4)
 * with the same encoders the synthesiser uses. */
int retro_b200_quantize_row(uint32_t ggml_type, const float * values, size_t n, uint8_t * out, size_t n_out, size_t * out_bytes);

/* Batch maps the GPU packing kernel built for the last step: tok_slot/tok_pos/tok_row/tok_cell
 * are `n_tokens` entries, out_index `n_out`, cu_rows `n_rows + 1`. Pass NULL to skip an array. */
int retro_b200_engine_last_pack(retro_engine * engine, size_t * n_tokens, size_t * n_out, int32_t * tok_slot,
                                int32_t * tok_pos, int32_t * tok_row, int32_t * tok_cell, int32_t * out_index,
                                int32_t * cu_rows, size_t capacity);
/* Logits row `index` (0-based among the sampling rows, row order) of the last step. */
int retro_b200_engine_last_logits(retro_engine * engine, size_t index, float * out, size_t n_vocab);
/* Expert ids chosen by the router in the last step: [layer][token][k], selection order. */
int retro_b200_engine_last_routes(retro_engine * engine, int32_t * out, size_t n_max, size_t * out_count);
/* Block table of a slot: physical block ids covering positions [0, pos_max]; the KV block
 * size (tokens per block) is written to *out_block_tokens. */
int retro_b200_engine_block_table(retro_engine * engine, int32_t slot, int32_t * out_blocks, size_t n_max,
                                  size_t * out_count, uint32_t * out_block_tokens);
/* Physical KV blocks in use (shared blocks counted once) and the total. */
int retro_b200_engine_blocks(retro_engine * engine, uint64_t * out_used, uint64_t * out_total);
/* Device time of the last step in milliseconds (CUDA events around its kernels) and the number
 * of kernels it launched. */
int retro_b200_engine_last_step_stats(retro_engine * engine, float * out_ms, uint64_t * out_launches);

/* One dequant-fused GEMM on host data: y[t][o] = sum_k deq(w)[o][k] * x[t][k] with w stored as
 * `ggml_type` rows. path: 0 engine's choice, 1 f32 row kernel, 3 exact
 * tensor-core kernel (mma.sync), 4 exact tcgen05 kernel, 5 exact weight-streaming
 * kernel (at most 8 tokens). Runs `iters` timed launches after one warm-up; *out_ms is the mean
 * device time per launch (operands smaller than 256 MB: a buffer larger than L2 is written before
 * every timed launch). */
int retro_b200_op_gemm(uint32_t ggml_type, const uint8_t * w, uint32_t n_out, uint32_t n_in, const float * x, uint32_t n_tokens, float * y,
                       int path, uint32_t iters, float * out_ms);

/* The grouped MXFP4 expert GEMM (tcgen05) on host data: `banks` = n_expert matrices of n_out rows x n_in
 * weights in 17-byte MXFP4 blocks, x = the offsets[n_expert] activation rows sorted by expert, offsets
 * [n_expert + 1] each expert's first row; y[r][o] = sum_k deq(bank[expert(r)])[o][k] * x[r][k]. -3 when the
 * operands are outside what the kernel covers (n_in % 64, block scales that are not f16 powers of two). `iters`
 * further launches are timed, each behind a write of a buffer larger than L2; *out_ms is their mean device time. */
int retro_b200_op_gemm_mxfp4_grouped(const uint8_t * banks, uint32_t n_expert, uint32_t n_out, uint32_t n_in, const float * x,
                                     const int32_t * offsets, float * y, uint32_t iters, float * out_ms);

/* No counterpart in the reference. The same exact Q4_K GEMM for callers that must not allocate
 * device memory (a host whose own pool owns the whole device budget, a loop that cannot take the
 * synchronisation an allocation may cause): d_w (Q4_K rows), d_x (f32 [n_tokens][n_in]) and d_y
 * (f32 [n_tokens][n_out]) are DEVICE pointers of the caller, `stream` its cudaStream_t or NULL. The
 * scratch the kernel needs lives in a fixed array inside the library (about 4.1 MiB per GPU that
 * loads it). Limit: n_tokens * n_in <= 1 048 576, n_in % 256 == 0; beyond it the call returns -3.
 * The first call on a device resolves the array's address on that device (a host-side lookup, no allocation).
 * All calls share the array, so calls that overlap on the GPU race; nothing needs clearing between
 * calls. The work is enqueued on `stream`; the call does not wait for it. */
int retro_b200_gemm_q4k_noalloc(const uint8_t * d_w, uint32_t n_out, uint32_t n_in, const float * d_x, uint32_t n_tokens, float * d_y,
                                void * stream);

/* Expert parallelism for mixture-of-experts models (the reference runs them on one GPU only:
 * src/runtime/retro_experts.cpp:86-140 places expert banks on a single device). One engine per GPU;
 * expert e is served by rank e / (n_expert / world). Rank 0 creates the 128-byte NCCL id, every rank
 * passes it to retro_b200_engine_ep_init (collective). Afterwards every MoE layer of every step
 * exchanges its (token, expert) pairs over NCCL, so all ranks must run the same number of steps; a rank
 * without rows calls retro_b200_engine_ep_idle_step instead. Results equal the single-GPU engine's.
 * retro_b200_ep_plan is the host arithmetic behind the exchange (all ranks' per-expert pair offsets
 * [world][n_expert + 1] -> what this rank sends, receives and how the received rows group by expert);
 * `sorted` needs room for *out_n_recv entries (-2 and the count when sorted_capacity is too small). */
int retro_b200_nccl_unique_id(void * out_id_128);
/* GGML type codes the layer's gate / up / down expert banks are held in on the device. MXFP4 banks (type 39)
 * stay MXFP4: the grouped tcgen05 GEMM decodes the 17-byte blocks itself when every block's E8M0 byte is in
 * 104..128 (every weight then is an f16); banks outside that range whose scales an f16 still holds are re-coded,
 * exactly, as Q8_0 (type 8) for the mma.sync grouped GEMM; RB200_MOE=rows keeps the CUDA-core row kernel. */
int retro_b200_engine_expert_storage(retro_engine * engine, int layer, uint32_t * out_types_3);
/* The load-time re-coding itself (host only, no GPU): n_blocks MXFP4 blocks (17 B each) -> Q8_0 blocks
 * (34 B each) holding the same values; *out_recoded = 0 and nothing written when a block's scale is not
 * a power of two an f16 holds (2^-24 .. 2^15). */
int retro_b200_recode_mxfp4_as_q8_0(const void * mxfp4, size_t n_blocks, void * out_q8_0, int * out_recoded);
int retro_b200_engine_ep_init(retro_engine * engine, int rank, int world, const void * unique_id_128);
int retro_b200_engine_ep_idle_step(retro_engine * engine);
int retro_b200_ep_plan(const int32_t * all_offsets, int world, int rank, int n_expert, int32_t * send_begin, int32_t * send_count,
                       int32_t * recv_begin, int32_t * recv_count, int32_t * offsets, int32_t * sorted, int32_t sorted_capacity,
                       int32_t * out_n_recv);

/* Bytes the last step copied host->device (the plan) and device->host (the sampled rows). */
int retro_b200_engine_last_step_io(retro_engine * engine, uint64_t * out_h2d_bytes, uint64_t * out_d2h_bytes);
/* Steps served so far by replaying a captured CUDA graph, and graphs currently cached. A step shape
 * (row count, token count, sampling rows, ...) seen twice is captured the second time and replayed
 * afterwards; profiling, MoE models and RB200_GRAPHS=0 keep every step eager. */
int retro_b200_engine_graph_stats(retro_engine * engine, uint64_t * out_replays, uint64_t * out_cached);
/* Per-class kernel timing with CUDA events on the launching stream. Classes, in order:
 * gemm, attention, sample, pack, moe, lora, other (RETRO_B200_PROFILE_CLASSES entries).
 * `enabled` switches the bracketing on or off, `reset` clears the accumulated totals. */
#define RETRO_B200_PROFILE_CLASSES 7
int retro_b200_engine_profile(retro_engine * engine, int enabled, int reset);
int retro_b200_engine_profile_read(retro_engine * engine, double * out_ms, uint64_t * out_launches, size_t n_classes);

#ifdef __cplusplus
}
#endif

#endif /* RETRO_B200_H */
