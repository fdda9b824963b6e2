// extern "C" surface of libretro_b200. Each entry point mirrors the reference entry point of the
// same name (crates/retrograd-ffi/runtime/src/retro_engine.cpp:454-1709): struct_size-prefixed
// config copy, validation messages, status codes, thread-local error, exception fence.

#include <cmath>
#include "engine.hpp"
#include "blocks.hpp"

#include <algorithm>
#include <climits>
#include <cstddef>
#include <cstring>

namespace rb200 {
uint64_t synth_gguf(const char * path, const char * spec_text);
size_t quantize_row(uint32_t type, const float * x, size_t n, uint8_t * out);
}

using namespace rb200;

// Layouts of the published header (crates/retrograd-ffi/src/lib.rs:2899-3052).
static_assert(sizeof(retro_engine_config) == 64 && alignof(retro_engine_config) == 8, "retro_engine_config layout");
static_assert(offsetof(retro_engine_config, n_ctx) == 4 && offsetof(retro_engine_config, n_seq_max) == 8 &&
              offsetof(retro_engine_config, n_batch) == 12 && offsetof(retro_engine_config, n_ubatch) == 16 &&
              offsetof(retro_engine_config, kv_dtype) == 20 && offsetof(retro_engine_config, flash_attn) == 24 &&
              offsetof(retro_engine_config, device) == 28 && offsetof(retro_engine_config, threads) == 32 &&
              offsetof(retro_engine_config, verbose) == 36 && offsetof(retro_engine_config, kv_unified) == 40 &&
              offsetof(retro_engine_config, expert_placement) == 44 && offsetof(retro_engine_config, expert_host_layers) == 48 &&
              offsetof(retro_engine_config, expert_device_cache_bytes) == 56, "retro_engine_config offsets");
static_assert(sizeof(retro_sampling_params) == 16, "retro_sampling_params layout");
static_assert(sizeof(retro_step_row) == 64 && alignof(retro_step_row) == 8, "retro_step_row layout");
static_assert(offsetof(retro_step_row, request) == 4 && offsetof(retro_step_row, slot) == 8 && offsetof(retro_step_row, tokens) == 16 &&
              offsetof(retro_step_row, n) == 24 && offsetof(retro_step_row, pos0) == 28 && offsetof(retro_step_row, sample) == 32 &&
              offsetof(retro_step_row, sampling) == 36 && offsetof(retro_step_row, n_top_logprobs) == 52 &&
              offsetof(retro_step_row, adapter) == 56, "retro_step_row offsets");
static_assert(sizeof(retro_step_out_row) == 20 && alignof(retro_step_out_row) == 4, "retro_step_out_row layout");
static_assert(offsetof(retro_step_out_row, token) == 4 && offsetof(retro_step_out_row, logprob) == 8 && offsetof(retro_step_out_row, n_top) == 12 &&
              offsetof(retro_step_out_row, forced) == 16 && offsetof(retro_step_out_row, sampled) == 17, "retro_step_out_row offsets");
static_assert(sizeof(retro_sampling_params_v2) == 72 && alignof(retro_sampling_params_v2) == 8, "retro_sampling_params_v2 layout");
static_assert(offsetof(retro_sampling_params_v2, temperature) == 4 && offsetof(retro_sampling_params_v2, top_p) == 8 &&
              offsetof(retro_sampling_params_v2, max_new_tokens) == 12 && offsetof(retro_sampling_params_v2, seed) == 16 &&
              offsetof(retro_sampling_params_v2, top_k) == 20 && offsetof(retro_sampling_params_v2, min_p) == 24 &&
              offsetof(retro_sampling_params_v2, repeat_penalty) == 28 && offsetof(retro_sampling_params_v2, frequency_penalty) == 32 &&
              offsetof(retro_sampling_params_v2, presence_penalty) == 36 && offsetof(retro_sampling_params_v2, penalty_window) == 40 &&
              offsetof(retro_sampling_params_v2, n_logit_bias) == 44 && offsetof(retro_sampling_params_v2, logit_bias_ids) == 48 &&
              offsetof(retro_sampling_params_v2, logit_bias_values) == 56 && offsetof(retro_sampling_params_v2, grammar) == 64,
              "retro_sampling_params_v2 offsets");
static_assert(sizeof(retro_step_row_v2) == 128 && alignof(retro_step_row_v2) == 8, "retro_step_row_v2 layout");
static_assert(offsetof(retro_step_row_v2, request) == 4 && offsetof(retro_step_row_v2, slot) == 8 && offsetof(retro_step_row_v2, tokens) == 16 &&
              offsetof(retro_step_row_v2, n) == 24 && offsetof(retro_step_row_v2, pos0) == 28 && offsetof(retro_step_row_v2, sample) == 32 &&
              offsetof(retro_step_row_v2, sampling) == 40 && offsetof(retro_step_row_v2, n_top_logprobs) == 112 &&
              offsetof(retro_step_row_v2, want_logprob) == 116 && offsetof(retro_step_row_v2, adapter) == 120, "retro_step_row_v2 offsets");
static_assert(sizeof(retro_step_out_row_v2) == 24 && offsetof(retro_step_out_row_v2, sampled_logprob) == 20, "retro_step_out_row_v2 layout");
static_assert(sizeof(retro_engine_memory_info) == 40 && offsetof(retro_engine_memory_info, n_slots) == 4 &&
              offsetof(retro_engine_memory_info, cells_total) == 8 && offsetof(retro_engine_memory_info, cells_used) == 16 &&
              offsetof(retro_engine_memory_info, kv_bytes) == 24 && offsetof(retro_engine_memory_info, recurrent_bytes) == 32,
              "retro_engine_memory_info layout");
static_assert(sizeof(retro_adapter_rows_info) == 32 && offsetof(retro_adapter_rows_info, n_adapters) == 4 &&
              offsetof(retro_adapter_rows_info, max_rank) == 8 && offsetof(retro_adapter_rows_info, stacked_bytes) == 16 &&
              offsetof(retro_adapter_rows_info, unpadded_bytes) == 24, "retro_adapter_rows_info layout");

namespace {

// Field values an absent config resolves to (retro_engine.cpp:93-110 lists the same numbers).
constexpr retro_engine_config kDefaultConfig = {
    /* struct_size */ sizeof(retro_engine_config), /* n_ctx */ 4096, /* n_seq_max */ 8, /* n_batch */ 512, /* n_ubatch */ 512,
    /* kv_dtype */ RETRO_ENGINE_KV_DTYPE_F16, /* flash_attn */ true, /* device */ RETRO_DEVICE_AUTO, /* threads */ 0, /* verbose */ false,
    /* kv_unified */ 1, /* expert_placement */ RETRO_EXPERT_PLACEMENT_DEVICE, /* expert_host_layers */ 0, /* expert_device_cache_bytes */ 0};

// Geometry rules of an engine config, in the order their messages are reported (the message texts and
// their order are the reference's contract, retro_engine.cpp:112-153; the first broken rule decides).
struct ConfigRule {
    bool (*broken)(const retro_engine_config &);
    const char * message;
};
constexpr ConfigRule kConfigRules[] = {
    {[](const retro_engine_config & c) { return c.n_ctx == 0 || c.n_seq_max == 0; }, "engine n_ctx and n_seq_max must be greater than zero"},
    {[](const retro_engine_config & c) { return c.n_batch == 0 || c.n_ubatch == 0 || c.n_ubatch > c.n_batch; }, "engine n_ubatch must be in (0, n_batch]"},
    {[](const retro_engine_config & c) { return std::max({c.n_ctx, c.n_batch, c.n_ubatch, c.threads}) > (uint32_t)INT32_MAX; },
     "engine context, batch and thread counts must fit in int32_t"},
    {[](const retro_engine_config & c) { return c.n_seq_max > std::min({kMaxSeq, c.n_batch, c.n_ctx}); },
     "engine n_seq_max must not exceed LLAMA_MAX_SEQ, n_batch or n_ctx"},
    {[](const retro_engine_config & c) { return c.kv_dtype < RETRO_ENGINE_KV_DTYPE_F32 || c.kv_dtype > RETRO_ENGINE_KV_DTYPE_Q4_0; },
     "engine kv_dtype must be one of retro_engine_kv_dtype"},
    {[](const retro_engine_config & c) { return c.kv_dtype >= RETRO_ENGINE_KV_DTYPE_Q8_0 && !c.flash_attn; }, "a quantized engine kv_dtype requires flash_attn"},
    {[](const retro_engine_config & c) { return c.device < RETRO_DEVICE_AUTO || c.device > RETRO_DEVICE_GPU; }, "engine device must be one of retro_device"},
    {[](const retro_engine_config & c) { return c.expert_placement != RETRO_EXPERT_PLACEMENT_DEVICE && c.expert_placement != RETRO_EXPERT_PLACEMENT_HOST; },
     "engine expert_placement must be one of retro_expert_placement"},
};

bool validate_engine_config(const retro_engine_config & c) {
    for (const ConfigRule & rule : kConfigRules) {
        if (!rule.broken(c)) continue;
        set_error(rule.message);
        return false;
    }
    return true;
}

Engine * checked(retro_engine * engine) {
    if (!engine) {
        set_error("engine handle is null");
        return nullptr;
    }
    return reinterpret_cast<Engine *>(engine);
}

bool is_blank(const char * s) {
    if (!s) return true;
    for (; *s; ++s) if (!isspace((unsigned char)*s)) return false;
    return true;
}

int write_string_out(const std::string & s, char * buffer, size_t n_buffer, size_t * out_n) {
    if (!out_n) {
        set_error("out_n_bytes is required");
        return STATUS_RUNTIME;
    }
    *out_n = s.size();
    if (!buffer || n_buffer == 0) return STATUS_OK;
    if (n_buffer < s.size()) {
        set_error("the output buffer is too small");
        return STATUS_BUFFER_TOO_SMALL;
    }
    std::memcpy(buffer, s.data(), s.size());
    return STATUS_OK;
}

int tokenize_into(Engine & e, const char * text, bool add_special, int32_t * tokens, size_t n_max, size_t * out_n) {
    if (!text || !out_n) {
        set_error("text and out_n_tokens are required");
        return STATUS_RUNTIME;
    }
    const Model & m = *e.model;
    // byte id lookup, built on first use from the `<0xNN>` pieces
    static thread_local const Model * cached = nullptr;
    static thread_local int32_t byte_id[256];
    if (cached != &m) {
        std::fill(byte_id, byte_id + 256, -1);
        for (size_t i = 0; i < m.vocab_tokens.size(); ++i) {
            const std::string & t = m.vocab_tokens[i];
            if (t.size() == 6 && t[0] == '<' && t[1] == '0' && t[2] == 'x' && t[5] == '>') byte_id[std::stoi(t.substr(3, 2), nullptr, 16)] = (int32_t)i;
        }
        cached = &m;
    }
    std::vector<int32_t> out;
    if (add_special && m.add_bos) out.push_back(m.bos);
    for (const unsigned char * p = (const unsigned char *)text; *p; ++p) {
        if (byte_id[*p] < 0) {
            set_error("the model's vocabulary has no byte-fallback pieces");
            return STATUS_RUNTIME;
        }
        out.push_back(byte_id[*p]);
    }
    *out_n = out.size();
    if (!tokens || n_max == 0) return STATUS_OK;
    if (n_max < out.size()) {
        set_error("the token buffer is too small");
        return STATUS_BUFFER_TOO_SMALL;
    }
    std::memcpy(tokens, out.data(), out.size() * 4);
    return STATUS_OK;
}

} // namespace

extern "C" {

const char * retro_last_error(void) { return last_error().c_str(); }

retro_engine * retro_engine_new(const char * model_path, const retro_engine_config * config) {
    return retro_engine_new_checked(model_path, config, nullptr);
}

retro_engine * retro_engine_new_checked(const char * model_path, const retro_engine_config * config, bool * out_invalid_placement) {
    if (out_invalid_placement) *out_invalid_placement = false;
    try {
        clear_error();
        if (is_blank(model_path)) {
            set_error("model_path is required");
            return nullptr;
        }
        retro_engine_config resolved = kDefaultConfig;
        if (config) {
            uint32_t size = 0;
            std::memcpy(&size, config, sizeof size);
            constexpr size_t required = offsetof(retro_engine_config, verbose) + sizeof(bool);
            if (size < required) {
                set_error("retro_engine_config.struct_size is too small for this build");
                return nullptr;
            }
            std::memcpy(&resolved, config, std::min<size_t>(size, sizeof resolved));
        }
        if (!validate_engine_config(resolved)) return nullptr;
        if (resolved.device == RETRO_DEVICE_CPU) {
            set_error("device=cpu requested but this library only runs on a CUDA GPU");
            return nullptr;
        }
        if (resolved.kv_dtype == RETRO_ENGINE_KV_DTYPE_F32) {
            set_error("this backend stores the KV cache as F16, Q8_0 or Q4_0: engine kv_dtype F32 is not supported");
            return nullptr;
        }
        if (resolved.expert_placement != RETRO_EXPERT_PLACEMENT_DEVICE) {
            if (out_invalid_placement) *out_invalid_placement = true;
            set_error("this backend keeps every expert bank in device memory: expert_placement must be DEVICE");
            return nullptr;
        }
        return reinterpret_cast<retro_engine *>(new Engine(model_path, resolved));
    } catch (const std::exception & err) {
        set_error(err.what());
        return nullptr;
    } catch (...) {
        set_error("unknown C++ exception");
        return nullptr;
    }
}

void retro_engine_free(retro_engine * engine) { delete reinterpret_cast<Engine *>(engine); }

int retro_engine_eos_token(retro_engine * engine, int32_t * out_token) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_token) {
            if (e) set_error("out_token is required");
            return STATUS_RUNTIME;
        }
        *out_token = e->model->eos;
        return STATUS_OK;
    });
}

int retro_engine_vocab_size(retro_engine * engine, uint32_t * out_n_vocab) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_n_vocab) {
            if (e) set_error("out_n_vocab is required");
            return STATUS_RUNTIME;
        }
        *out_n_vocab = e->model->hp.vocab;
        return STATUS_OK;
    });
}

int retro_engine_is_eog_token(retro_engine * engine, int32_t token, bool * out_is_eog) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_is_eog) {
            if (e) set_error("out_is_eog is required");
            return STATUS_RUNTIME;
        }
        if (token < 0 || (uint32_t)token >= e->model->hp.vocab) {
            set_error("token is outside the vocabulary");
            return STATUS_RUNTIME;
        }
        *out_is_eog = e->model->is_eog(token);
        return STATUS_OK;
    });
}

int retro_engine_context_size(retro_engine * engine, uint32_t * out_n_ctx) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_n_ctx) {
            if (e) set_error("out_n_ctx is required");
            return STATUS_RUNTIME;
        }
        *out_n_ctx = e->n_ctx_seq;
        return STATUS_OK;
    });
}

int retro_engine_detokenize(retro_engine * engine, const int32_t * tokens, size_t n_tokens, bool unparse_special, char * buffer,
                            size_t n_buffer, size_t * out_n_bytes) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!out_n_bytes) {
            set_error("out_n_bytes is required");
            return STATUS_RUNTIME;
        }
        if (n_tokens > 0 && !tokens) {
            set_error("tokens are required");
            return STATUS_RUNTIME;
        }
        std::string text;
        for (size_t i = 0; i < n_tokens; ++i) {
            if (tokens[i] < 0 || (uint32_t)tokens[i] >= e->model->hp.vocab) {
                set_error("token is outside the vocabulary");
                return STATUS_RUNTIME;
            }
            text += e->model->piece(tokens[i], unparse_special);
        }
        return write_string_out(text, buffer, n_buffer, out_n_bytes);
    });
}

int retro_engine_tokenize_text(retro_engine * engine, const char * text, int32_t * tokens, size_t n_tokens_max, size_t * out_n_tokens) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        return tokenize_into(*e, text, true, tokens, n_tokens_max, out_n_tokens);
    });
}

int retro_engine_tokenize_fragment(retro_engine * engine, const char * text, int32_t * tokens, size_t n_tokens_max, size_t * out_n_tokens) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        return tokenize_into(*e, text, false, tokens, n_tokens_max, out_n_tokens);
    });
}

int retro_engine_adapter_load(retro_engine * engine, const char * adapter_path, float scale, int32_t * out_id) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        return e->adapter_load(adapter_path, scale, out_id);
    });
}

int retro_engine_adapter_unload(retro_engine * engine, int32_t id) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        return e->adapter_unload(id);
    });
}

int retro_engine_adapter_rows_info(retro_engine * engine, retro_adapter_rows_info * out_info) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_info) {
            if (e) set_error("out_info is required");
            return STATUS_RUNTIME;
        }
        e->adapter_info(out_info);
        return STATUS_OK;
    });
}

int retro_engine_graphs_reused(retro_engine * engine, uint64_t * out_n_reused) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_n_reused) {
            if (e) set_error("out_n_reused is required");
            return STATUS_RUNTIME;
        }
        *out_n_reused = e->graphs_reused;
        return STATUS_OK;
    });
}

int retro_engine_step(retro_engine * engine, const retro_step_row * rows, size_t n_rows, retro_step_out_row * out_rows,
                      int32_t * out_top_ids, float * out_top_logprobs, size_t n_top_stride) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!rows || n_rows == 0 || !out_rows) {
            set_error("step rows and output rows are required");
            return STATUS_INVALID_ARGUMENT;
        }
        std::vector<EffRow> eff(n_rows);
        for (size_t r = 0; r < n_rows; ++r) {
            const retro_step_row & row = rows[r];
            if (row.struct_size < offsetof(retro_step_row, adapter) + sizeof(int32_t)) {
                set_error("retro_step_row.struct_size is too small for this build");
                return STATUS_INVALID_ARGUMENT;
            }
            eff[r] = EffRow{row.struct_size, row.request, row.slot, row.tokens, row.n, row.pos0, row.sample, row.sampling, nullptr,
                            row.n_top_logprobs, false, row.adapter};
        }
        std::vector<OutRow> internal(n_rows);
        const int status = e->step(eff.data(), n_rows, internal.data(), out_top_ids, out_top_logprobs, n_top_stride);
        if (status != 0) return status;
        for (size_t r = 0; r < n_rows; ++r) {
            retro_step_out_row & o = out_rows[r];
            o.struct_size = sizeof(retro_step_out_row);
            o.token = internal[r].token;
            o.logprob = internal[r].logprob;
            o.n_top = internal[r].n_top;
            o.forced = internal[r].forced;
            o.sampled = internal[r].sampled;
        }
        return STATUS_OK;
    });
}

int retro_engine_step_v2(retro_engine * engine, const retro_step_row_v2 * rows, size_t n_rows, retro_step_out_row_v2 * out_rows,
                         int32_t * out_top_ids, float * out_top_logprobs, size_t n_top_stride) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!rows || n_rows == 0 || !out_rows) {
            set_error("step rows and output rows are required");
            return STATUS_INVALID_ARGUMENT;
        }
        std::vector<EffRow> eff(n_rows);
        for (size_t r = 0; r < n_rows; ++r) {
            const retro_step_row_v2 & row = rows[r];
            if (row.struct_size < offsetof(retro_step_row_v2, adapter) + sizeof(int32_t)) {
                set_error("retro_step_row_v2.struct_size is too small for this build");
                return STATUS_INVALID_ARGUMENT;
            }
            if (row.sampling.struct_size < sizeof(retro_sampling_params_v2)) {
                set_error("retro_sampling_params_v2.struct_size is too small for this build");
                return STATUS_INVALID_ARGUMENT;
            }
            eff[r] = EffRow{row.struct_size, row.request, row.slot, row.tokens, row.n, row.pos0, row.sample, retro_sampling_params{},
                            &row.sampling, row.n_top_logprobs, row.want_logprob != 0, row.adapter};
        }
        std::vector<OutRow> internal(n_rows);
        const int status = e->step(eff.data(), n_rows, internal.data(), out_top_ids, out_top_logprobs, n_top_stride);
        if (status != 0) return status;
        for (size_t r = 0; r < n_rows; ++r) {
            retro_step_out_row_v2 & o = out_rows[r];
            o.struct_size = sizeof(retro_step_out_row_v2);
            o.token = internal[r].token;
            o.logprob = internal[r].logprob;
            o.n_top = internal[r].n_top;
            o.forced = internal[r].forced;
            o.sampled = internal[r].sampled;
            o.sampled_logprob = internal[r].sampled_logprob;
        }
        return STATUS_OK;
    });
}

int retro_engine_seq_rm(retro_engine * engine, int32_t slot, int32_t p0, int32_t p1) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->seq_rm(slot, p0, p1) : STATUS_RUNTIME;
    });
}

int retro_engine_seq_cp(retro_engine * engine, int32_t src, int32_t dst, int32_t p0, int32_t p1) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->seq_cp(src, dst, p0, p1) : STATUS_RUNTIME;
    });
}

int retro_engine_seq_save(retro_engine * engine, int32_t slot, uint32_t flags, uint8_t * buffer, size_t n_buffer, size_t * out_n_bytes) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->seq_save(slot, flags, buffer, n_buffer, out_n_bytes) : STATUS_RUNTIME;
    });
}

int retro_engine_seq_load(retro_engine * engine, int32_t slot, uint32_t flags, const uint8_t * buffer, size_t n_bytes, size_t * out_n_read) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->seq_load(slot, flags, buffer, n_bytes, out_n_read) : STATUS_RUNTIME;
    });
}

int retro_engine_seq_pos(retro_engine * engine, int32_t slot, int32_t * out_pos_min, int32_t * out_pos_max) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->seq_pos(slot, out_pos_min, out_pos_max) : STATUS_RUNTIME;
    });
}

int retro_engine_memory(retro_engine * engine, retro_engine_memory_info * out) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->memory(out) : STATUS_RUNTIME;
    });
}

namespace {

bool valid_v1_sampling(const retro_sampling_params & s) {
    if (!(s.temperature > 0.0f) || !std::isfinite(s.temperature)) {
        set_error("sampling temperature must be finite and greater than zero");
        return false;
    }
    if (!(s.top_p > 0.0f && s.top_p <= 1.0f)) {
        set_error("sampling top_p must be in (0, 1]");
        return false;
    }
    if (s.max_new_tokens == 0) {
        set_error("sampling max_new_tokens must be greater than zero");
        return false;
    }
    return true;
}

struct GenItem {
    const int32_t * prompt;
    size_t n_prompt;
    retro_sampling_params sampling;
};

// The shared loop of both generators. `shared_prompt`: every item has the same prompt; it is decoded
// once into slot 0 up to its last token, and the other slots share those cells (seq_cp).
int generate_over_steps(Engine * e, const std::vector<GenItem> & items, bool shared_prompt, int32_t * out_tokens, float * out_logprobs,
                        size_t n_out_max, size_t * out_n_tokens, uint8_t * out_forced) {
    const size_t n = items.size();
    const size_t n_batch = e->config.n_batch, n_ctx = e->n_ctx_seq;
    const int32_t request_base = 0x40000000;             // ids of this call's rows; freed before returning
    auto forget = [&]() {
        for (size_t i = 0; i < e->config.n_seq_max; ++i) e->seq_rm((int32_t)i, -1, -1);
        for (size_t i = 0; i < n; ++i) e->requests.erase(request_base + (int32_t)i);
    };
    forget();
    GenerationCounters & stats = e->gen_stats;
    stats.calls += 1;
    stats.sequences += n;
    for (size_t i = 0; i < n; ++i) stats.prompt_tokens += items[i].n_prompt;
    std::vector<size_t> limit(n), fed(n, 0);
    std::vector<int32_t> last(n, 0);
    std::vector<bool> live(n, true);
    for (size_t i = 0; i < n; ++i) {
        limit[i] = std::min<size_t>(std::min<size_t>(n_out_max, items[i].sampling.max_new_tokens), n_ctx - items[i].n_prompt);
        out_n_tokens[i] = 0;
    }
    std::vector<EffRow> rows;
    std::vector<OutRow> outs;
    std::vector<size_t> row_item;
    auto run = [&]() -> int {
        outs.assign(rows.size(), OutRow{});
        return e->step(rows.data(), rows.size(), outs.data(), nullptr, nullptr, 0);
    };
    auto row_of = [&](size_t i, const int32_t * tokens, size_t count, size_t pos0, bool sample) {
        EffRow r{};
        r.struct_size = sizeof(retro_step_row);
        r.request = request_base + (int32_t)i;
        r.slot = (int32_t)i;
        r.tokens = tokens;
        r.n = (uint32_t)count;
        r.pos0 = (int32_t)pos0;
        r.sample = sample;
        r.v1 = items[i].sampling;
        r.v2 = nullptr;
        r.n_top_logprobs = 0;
        r.want_logprob = false;
        r.adapter = 0;
        return r;
    };
    auto record = [&](size_t i, const OutRow & o) {
        const size_t count = out_n_tokens[i];
        out_tokens[i * n_out_max + count] = o.token;
        if (out_logprobs) out_logprobs[i * n_out_max + count] = o.logprob;
        if (out_forced) out_forced[i * n_out_max + count] = 0;
        out_n_tokens[i] = count + 1;
        last[i] = o.token;
        if (e->model->is_eog(o.token) || out_n_tokens[i] == limit[i]) live[i] = false;
    };

    // ---- prompts
    if (shared_prompt) {
        const GenItem & it = items[0];
        for (size_t pos = 0; pos + 1 < it.n_prompt;) {          // everything but the last token, into slot 0
            const size_t take = std::min(n_batch, it.n_prompt - 1 - pos);
            rows.assign(1, row_of(0, it.prompt + pos, take, pos, false));
            const int st = run();
            if (st != 0) { forget(); return st; }
            pos += take;
            stats.prefilled_tokens += take;
        }
        if (it.n_prompt > 1)
            for (size_t i = 1; i < n; ++i) {
                // slot 0 holds exactly [0, n_prompt - 2]: the whole-sequence form says the same and is the only
                // one a partitioned pool accepts
                const int st = e->seq_cp(0, (int32_t)i, -1, -1);
                if (st != 0) { forget(); return st; }
                stats.hits += 1;
                stats.reused_tokens += it.n_prompt - 1;
            }
        for (size_t i = 0; i < n; ++i) fed[i] = it.n_prompt - 1;
    }
    // remaining prompt tokens in chunks, several sequences per step while the token budget lasts;
    // the row that carries a prompt's last token samples
    while (true) {
        rows.clear();
        row_item.clear();
        size_t budget = n_batch;
        for (size_t i = 0; i < n && budget > 0; ++i) {
            if (fed[i] >= items[i].n_prompt) continue;
            const size_t take = std::min(budget, items[i].n_prompt - fed[i]);
            rows.push_back(row_of(i, items[i].prompt + fed[i], take, fed[i], fed[i] + take == items[i].n_prompt));
            row_item.push_back(i);
            budget -= take;
        }
        if (rows.empty()) break;
        const int st = run();
        if (st != 0) { forget(); return st; }
        for (size_t r = 0; r < rows.size(); ++r) {
            const size_t i = row_item[r];
            fed[i] += rows[r].n;
            stats.prefilled_tokens += rows[r].n;
            if (rows[r].sample) record(i, outs[r]);
        }
    }
    // ---- decode: every live sequence feeds its last token back
    while (true) {
        rows.clear();
        row_item.clear();
        for (size_t i = 0; i < n; ++i) {
            if (!live[i]) continue;
            rows.push_back(row_of(i, &last[i], 1, items[i].n_prompt + out_n_tokens[i] - 1, true));
            row_item.push_back(i);
        }
        if (rows.empty()) break;
        const int st = run();
        if (st != 0) { forget(); return st; }
        for (size_t r = 0; r < rows.size(); ++r) record(row_item[r], outs[r]);
    }
    forget();
    return STATUS_OK;
}

} // namespace

int retro_engine_generate_batch(retro_engine * engine, const int32_t * prompt_tokens, size_t n_prompt, const retro_sampling_params * sampling,
                                size_t n_sequences, int32_t * out_tokens, float * out_logprobs, size_t n_out_max, size_t * out_n_tokens,
                                uint8_t * out_forced) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!prompt_tokens || n_prompt == 0) {
            set_error("prompt tokens are required");
            return STATUS_RUNTIME;
        }
        if (!sampling || n_sequences == 0 || !out_tokens || !out_n_tokens || n_out_max == 0) {
            set_error("sampling params and output buffers are required");
            return STATUS_RUNTIME;
        }
        if (n_sequences > e->config.n_seq_max) {
            set_error("generation batch has " + std::to_string(n_sequences) + " sequences but the context supports " +
                      std::to_string(e->config.n_seq_max));
            return STATUS_RUNTIME;
        }
        if (n_sequences > e->config.n_batch) {
            set_error("generation batch exceeds the configured batch capacity");
            return STATUS_RUNTIME;
        }
        if (n_sequences > SIZE_MAX / n_out_max) {
            set_error("generation batch output shape overflows size_t");
            return STATUS_RUNTIME;
        }
        for (size_t i = 0; i < n_sequences; ++i)
            if (!valid_v1_sampling(sampling[i])) return STATUS_RUNTIME;
        for (size_t i = 0; i < n_prompt; ++i)
            if (prompt_tokens[i] < 0 || (uint32_t)prompt_tokens[i] >= e->model->hp.vocab) {
                set_error("token id " + std::to_string(prompt_tokens[i]) + " is outside the vocabulary");
                return STATUS_RUNTIME;
            }
        if (n_prompt >= e->n_ctx_seq) {
            set_error("prompt of " + std::to_string(n_prompt) + " tokens leaves no room to generate in context " + std::to_string(e->n_ctx_seq));
            return STATUS_RUNTIME;
        }
        std::vector<GenItem> items(n_sequences);
        for (size_t i = 0; i < n_sequences; ++i) items[i] = GenItem{prompt_tokens, n_prompt, sampling[i]};
        return generate_over_steps(e, items, true, out_tokens, out_logprobs, n_out_max, out_n_tokens, out_forced);
    });
}

int retro_engine_generate_continuous_batch(retro_engine * engine, const retro_generation_sequence * sequences, size_t n_sequences,
                                           int32_t * out_tokens, float * out_logprobs, size_t n_out_max, size_t * out_n_tokens,
                                           uint8_t * out_forced) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!sequences || n_sequences == 0 || !out_tokens || !out_n_tokens || n_out_max == 0) {
            set_error("continuous generation inputs and output buffers are required");
            return STATUS_RUNTIME;
        }
        if (n_sequences > e->config.n_seq_max || n_sequences > e->config.n_batch) {
            set_error("continuous generation batch exceeds the configured sequence or batch capacity");
            return STATUS_RUNTIME;
        }
        if (n_sequences > SIZE_MAX / n_out_max) {
            set_error("continuous generation output shape overflows size_t");
            return STATUS_RUNTIME;
        }
        std::vector<GenItem> items(n_sequences);
        for (size_t i = 0; i < n_sequences; ++i) {
            const retro_generation_sequence & s = sequences[i];
            bool ok = s.prompt_tokens && s.n_prompt > 0 && s.n_prompt < e->n_ctx_seq;
            set_error("");
            if (ok) ok = valid_v1_sampling(s.sampling);
            for (size_t k = 0; ok && k < s.n_prompt; ++k) ok = s.prompt_tokens[k] >= 0 && (uint32_t)s.prompt_tokens[k] < e->model->hp.vocab;
            if (!ok) {
                if (std::string(retro_last_error()).empty()) set_error("invalid continuous generation prompt");
                return STATUS_RUNTIME;
            }
            items[i] = GenItem{s.prompt_tokens, s.n_prompt, s.sampling};
        }
        return generate_over_steps(e, items, false, out_tokens, out_logprobs, n_out_max, out_n_tokens, out_forced);
    });
}

int retro_engine_request_free(retro_engine * engine, int32_t request) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        e->requests.erase(request);
        return STATUS_OK;
    });
}

int retro_engine_kv_unified(retro_engine * engine, bool * out_unified) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_unified) {
            if (e) set_error("out_unified is required");
            return STATUS_RUNTIME;
        }
        *out_unified = e->config.kv_unified != 0;
        return STATUS_OK;
    });
}

int retro_engine_weights_version(retro_engine * engine, uint64_t * out_version) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_version) {
            if (e) set_error("out_version is required");
            return STATUS_RUNTIME;
        }
        *out_version = e->weights_version;
        return STATUS_OK;
    });
}

int retro_engine_model_fingerprint(retro_engine * engine, uint64_t * out_fingerprint) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_fingerprint) {
            if (e) set_error("out_fingerprint is required");
            return STATUS_RUNTIME;
        }
        *out_fingerprint = e->fingerprint;
        return STATUS_OK;
    });
}

int retro_engine_is_hybrid(retro_engine * engine, bool * out_is_hybrid) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_is_hybrid) {
            if (e) set_error("out_is_hybrid is required");
            return STATUS_RUNTIME;
        }
        *out_is_hybrid = false;
        return STATUS_OK;
    });
}

int retro_engine_expert_route_enable(retro_engine * engine, uint32_t sample_every) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        e->route_enabled = sample_every != 0;
        return STATUS_OK;
    });
}

int retro_engine_expert_route_counts(retro_engine * engine, uint32_t layer, uint32_t * out, size_t n_expert) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out) {
            if (e) set_error("out is required");
            return STATUS_RUNTIME;
        }
        if (layer >= e->route_counts.size() || n_expert < e->model->hp.n_expert) {
            set_error("layer or expert count is outside the model's MoE geometry");
            return STATUS_RUNTIME;
        }
        std::memcpy(out, e->route_counts[layer].data(), e->model->hp.n_expert * 4);
        return STATUS_OK;
    });
}

int retro_engine_expert_route_reset(retro_engine * engine) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        for (auto & l : e->route_counts) std::fill(l.begin(), l.end(), 0u);
        return STATUS_OK;
    });
}

// ---- serialised adapters ---------------------------------------------------------------------

int retro_engine_load_lora(retro_engine * engine, const char * adapter_path) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (is_blank(adapter_path)) {
            set_error("adapter_path is required");
            return STATUS_RUNTIME;
        }
        return e->lora_load_single(adapter_path);
    });
}

int retro_engine_load_lora_named(retro_engine * engine, const char * name, const char * adapter_path) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (is_blank(name)) {
            set_error("name is required");
            return STATUS_RUNTIME;
        }
        if (is_blank(adapter_path)) {
            set_error("adapter_path is required");
            return STATUS_RUNTIME;
        }
        return e->lora_load_named(name, adapter_path);
    });
}

int retro_engine_activate_lora(retro_engine * engine, const char * name) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->lora_activate(name) : STATUS_RUNTIME;
    });
}

int retro_engine_set_lora_enabled(retro_engine * engine, bool enabled) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->lora_set_enabled(enabled) : STATUS_RUNTIME;
    });
}

namespace {
// The two-call text contract of the reference's string outputs (retro_runtime.hpp:551-576): without a
// buffer only the length is reported; with one, the text and a terminating NUL must fit.
int text_out(const std::string & text, char * buffer, size_t n_buffer, size_t * out_n_bytes) {
    *out_n_bytes = text.size();
    if (!buffer || n_buffer == 0) return STATUS_OK;
    if (text.size() > n_buffer - 1) {
        set_error("output buffer is too small");
        return STATUS_BUFFER_TOO_SMALL;
    }
    std::memcpy(buffer, text.data(), text.size());
    buffer[text.size()] = '\0';
    return STATUS_OK;
}
} // namespace

int retro_engine_active_adapter(retro_engine * engine, char * buffer, size_t n_buffer, size_t * out_n_bytes) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!out_n_bytes) {
            set_error("out_n_bytes is required");
            return STATUS_RUNTIME;
        }
        return text_out(e->active_adapter(), buffer, n_buffer, out_n_bytes);
    });
}

// ---- counters and memory ---------------------------------------------------------------------

static_assert(sizeof(retro_memory_report) == 216 && alignof(retro_memory_report) == 8 && offsetof(retro_memory_report, trainable_parameter_bytes) == 48 &&
              offsetof(retro_memory_report, base_trainable_on_host) == 74 && offsetof(retro_memory_report, device_bytes) == 80 &&
              offsetof(retro_memory_report, device_memory_samples) == 136, "retro_memory_report layout");
static_assert(sizeof(retro_generation_stats) == 56, "retro_generation_stats layout");
static_assert(sizeof(retro_expert_bank_desc) == 272 && offsetof(retro_expert_bank_desc, role) == 4 && offsetof(retro_expert_bank_desc, tensor) == 24,
              "retro_expert_bank_desc layout");
static_assert(sizeof(retro_expert_cache_stats) == 464 && offsetof(retro_expert_cache_stats, n_groups) == 72 && offsetof(retro_expert_cache_stats, groups) == 80,
              "retro_expert_cache_stats layout");

int retro_engine_memory_report(retro_engine * engine, retro_memory_report * out_report) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_report) {
            if (e) set_error("out_report is required");
            return STATUS_RUNTIME;
        }
        retro_memory_report r{};
        r.has_generation_context = true;
        r.model_weight_bytes = e->model->weight_bytes + e->model->tiled_bytes;
        retro_engine_memory_info kv{};
        e->memory(&kv);
        r.generation_kv_bytes = kv.kv_bytes;
        r.generation_compute_bytes = e->work_buffer_bytes();
        r.trainable_parameter_bytes = e->adapter_bytes();
        r.trainable_parameters_are_model_subset = false;
        r.adapter_on_host = false;
        r.base_trainable_on_host = false;
        r.device_bytes = r.model_weight_bytes + r.generation_kv_bytes + r.generation_compute_bytes + r.trainable_parameter_bytes;
        size_t free_bytes = 0, total_bytes = 0;
        if (cudaMemGetInfo(&free_bytes, &total_bytes) == cudaSuccess) {
            r.device_total_bytes = total_bytes;
            r.device_used_bytes = total_bytes - free_bytes;
            r.device_peak_used_bytes = r.device_used_bytes;
            r.backend_scratch_bytes = r.device_used_bytes > r.device_bytes ? r.device_used_bytes - r.device_bytes : 0;
            r.backend_scratch_peak_bytes = r.backend_scratch_bytes;
            r.device_memory_samples = 1;
        } else {
            cudaGetLastError();
        }
        *out_report = r;
        return STATUS_OK;
    });
}

int retro_engine_generation_stats(retro_engine * engine, retro_generation_stats * out_stats) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_stats) {
            if (e) set_error("out_stats is required");
            return STATUS_RUNTIME;
        }
        const GenerationCounters & c = e->gen_stats;
        *out_stats = retro_generation_stats{c.calls, c.sequences, c.prompt_tokens, c.prefilled_tokens, c.reused_tokens, c.hits, c.evictions};
        return STATUS_OK;
    });
}

// ---- expert banks ----------------------------------------------------------------------------

int retro_engine_expert_banks(retro_engine * engine, retro_expert_bank_desc * out_banks, size_t n_max, size_t * out_count) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!out_count) {
            set_error("out_count is required");
            return STATUS_RUNTIME;
        }
        const std::vector<retro_expert_bank_desc> & banks = e->model->expert_banks;
        *out_count = banks.size();
        if (!out_banks || banks.empty()) return STATUS_OK;
        if (n_max < banks.size()) {
            set_error("expert bank buffer is too small");
            return STATUS_BUFFER_TOO_SMALL;
        }
        std::copy(banks.begin(), banks.end(), out_banks);
        return STATUS_OK;
    });
}

int retro_engine_expert_stats(retro_engine * engine, retro_expert_cache_stats * out_stats) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_stats) {
            if (e) set_error("out_stats is required");
            return STATUS_RUNTIME;
        }
        *out_stats = retro_expert_cache_stats{};      // no device cache: every bank is resident
        return STATUS_OK;
    });
}

int retro_engine_expert_route_paths(retro_engine * engine, uint64_t out[3]) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out) {
            if (e) set_error("routing paths output is required");
            return STATUS_RUNTIME;
        }
        out[0] = e->route_pairs;
        out[1] = 0;
        out[2] = 0;
        return STATUS_OK;
    });
}

// ---- grammar handles: host-only owners of a GBNF text (retro_grammar.cpp:1-76) --------------------

} // extern "C"

namespace {
// Any JSON object, in GBNF. Written for this library (the reference embeds its fork's grammar file).
const char kJsonObjectGbnf[] =
    "root ::= object\n"
    "value ::= object | array | string | number | (\"true\" | \"false\" | \"null\") ws\n"
    "object ::= \"{\" ws ( member (\",\" ws member)* )? \"}\" ws\n"
    "member ::= string \":\" ws value\n"
    "array ::= \"[\" ws ( value (\",\" ws value)* )? \"]\" ws\n"
    "string ::= \"\\\"\" ( [^\"\\\\\\x7F\\x00-\\x1F] | \"\\\\\" ( [\"\\\\/bfnrt] | \"u\" [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F] ) )* \"\\\"\" ws\n"
    "number ::= \"-\"? ( \"0\" | [1-9] [0-9]* ) ( \".\" [0-9]+ )? ( [eE] [-+]? [0-9]+ )? ws\n"
    "ws ::= [ \\t\\n\\r]*\n";

retro_grammar * grammar_of(const char * text, const char * what) {
    retro_grammar * result = nullptr;
    boundary([&]() -> int {
        if (!text || text[0] == '\0') {
            set_error(std::string(what) + " is required and must not be empty");
            return STATUS_RUNTIME;
        }
        result = new retro_grammar{std::string(text)};
        return STATUS_OK;
    });
    return result;
}
} // namespace

extern "C" {

retro_grammar * retro_grammar_from_gbnf(const char * gbnf) { return grammar_of(gbnf, "gbnf"); }

retro_grammar * retro_grammar_json_object(void) { return grammar_of(kJsonObjectGbnf, "gbnf"); }

retro_grammar * retro_grammar_from_json_schema(const char * json_schema) {
    if (!json_schema || json_schema[0] == '\0') {
        set_error("json_schema is required and must not be empty");
        return nullptr;
    }
    set_error("this library does not convert JSON schemas to grammars (the converter belongs to the reference's llama.cpp fork): pass GBNF to "
              "retro_grammar_from_gbnf");
    return nullptr;
}

const char * retro_grammar_gbnf(const retro_grammar * grammar) {
    if (!grammar) {
        set_error("grammar is null");
        return nullptr;
    }
    return grammar->gbnf.c_str();
}

void retro_grammar_free(retro_grammar * grammar) { delete grammar; }

// Host-only: how a text stands in a grammar. *out_state = 0 rejected, 1 a valid prefix, 2 complete (the whole
// text matches the root rule). -3 with the parser's message for an invalid grammar.
int retro_b200_grammar_check(const char * gbnf, const char * text, int * out_state) {
    return boundary([&]() -> int {
        if (!gbnf || !text || !out_state) {
            set_error("gbnf, text and out_state are required");
            return STATUS_INVALID_ARGUMENT;
        }
        try {
            GrammarState state;
            state.grammar = std::make_shared<const Grammar>(gbnf);
            state.stacks = state.grammar->initial();
            if (!state.advance(text, false) || !state.pending.empty()) {
                *out_state = 0;
            } else {
                *out_state = Grammar::complete(state.stacks) ? 2 : 1;
            }
        } catch (const std::invalid_argument & err) {
            set_error(err.what());
            return STATUS_INVALID_ARGUMENT;
        }
        return STATUS_OK;
    });
}

// ---- the trainer-owned generation context ------------------------------------------------------
// A retro_trainer made here owns one generation context and nothing else; every twin forwards to the
// engine entry point of the same contract.

} // extern "C"

struct retro_trainer {
    retro_engine * generation = nullptr;
};

namespace {
retro_engine * generation_of(retro_trainer * trainer) {
    if (!trainer || !trainer->generation) {
        set_error("trainer handle is null");
        return nullptr;
    }
    return trainer->generation;
}
} // namespace

extern "C" {

retro_trainer * retro_b200_trainer_generation_new(const char * model_path, const retro_engine_config * config, const char * adapter_path) {
    retro_engine * engine = retro_engine_new(model_path, config);
    if (!engine) return nullptr;
    if (adapter_path && retro_engine_load_lora(engine, adapter_path) != 0) {
        retro_engine_free(engine);
        return nullptr;
    }
    return new retro_trainer{engine};
}

void retro_b200_trainer_generation_free(retro_trainer * trainer) {
    if (!trainer) return;
    retro_engine_free(trainer->generation);
    delete trainer;
}

// The weights behind the generation context changed (an optimizer step, a weight import): with a path the
// trained adapter is read again, and either way the KV is forgotten and the weights version moves on.
int retro_b200_trainer_weights_updated(retro_trainer * trainer, const char * adapter_path) {
    retro_engine * g = generation_of(trainer);
    if (!g) return STATUS_RUNTIME;
    if (adapter_path) return retro_engine_load_lora(g, adapter_path);
    return boundary([&]() -> int {
        reinterpret_cast<Engine *>(g)->forget_kv();
        return STATUS_OK;
    });
}

int retro_trainer_generation_step(retro_trainer * trainer, const retro_step_row * rows, size_t n_rows, retro_step_out_row * out_rows,
                                  int32_t * out_top_ids, float * out_top_logprobs, size_t n_top_stride) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_step(g, rows, n_rows, out_rows, out_top_ids, out_top_logprobs, n_top_stride) : STATUS_RUNTIME;
}
int retro_trainer_generation_step_v2(retro_trainer * trainer, const retro_step_row_v2 * rows, size_t n_rows, retro_step_out_row_v2 * out_rows,
                                     int32_t * out_top_ids, float * out_top_logprobs, size_t n_top_stride) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_step_v2(g, rows, n_rows, out_rows, out_top_ids, out_top_logprobs, n_top_stride) : STATUS_RUNTIME;
}
int retro_trainer_generation_seq_rm(retro_trainer * trainer, int32_t slot, int32_t p0, int32_t p1) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_seq_rm(g, slot, p0, p1) : STATUS_RUNTIME;
}
int retro_trainer_generation_seq_cp(retro_trainer * trainer, int32_t src, int32_t dst, int32_t p0, int32_t p1) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_seq_cp(g, src, dst, p0, p1) : STATUS_RUNTIME;
}
int retro_trainer_generation_seq_save(retro_trainer * trainer, int32_t slot, uint32_t flags, uint8_t * buffer, size_t n_buffer, size_t * out_n_bytes) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_seq_save(g, slot, flags, buffer, n_buffer, out_n_bytes) : STATUS_RUNTIME;
}
int retro_trainer_generation_seq_load(retro_trainer * trainer, int32_t slot, uint32_t flags, const uint8_t * buffer, size_t n_bytes, size_t * out_n_read) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_seq_load(g, slot, flags, buffer, n_bytes, out_n_read) : STATUS_RUNTIME;
}
int retro_trainer_generation_seq_pos(retro_trainer * trainer, int32_t slot, int32_t * out_pos_min, int32_t * out_pos_max) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_seq_pos(g, slot, out_pos_min, out_pos_max) : STATUS_RUNTIME;
}
int retro_trainer_generation_memory(retro_trainer * trainer, retro_engine_memory_info * out) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_memory(g, out) : STATUS_RUNTIME;
}
int retro_trainer_generation_request_free(retro_trainer * trainer, int32_t request) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_request_free(g, request) : STATUS_RUNTIME;
}
int retro_trainer_generation_kv_unified(retro_trainer * trainer, bool * out_unified) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_kv_unified(g, out_unified) : STATUS_RUNTIME;
}
int retro_trainer_generation_weights_version(retro_trainer * trainer, uint64_t * out_version) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_weights_version(g, out_version) : STATUS_RUNTIME;
}
int retro_trainer_generation_stats(retro_trainer * trainer, retro_generation_stats * out_stats) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_generation_stats(g, out_stats) : STATUS_RUNTIME;
}
int retro_trainer_generation_adapter_snapshot(retro_trainer * trainer, int32_t replace, float scale, int32_t * out_id) {
    retro_engine * g = generation_of(trainer);
    if (!g) return STATUS_RUNTIME;
    return boundary([&]() -> int { return reinterpret_cast<Engine *>(g)->adapter_snapshot(replace, scale, out_id); });
}
int retro_trainer_generation_adapter_unload(retro_trainer * trainer, int32_t id) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_adapter_unload(g, id) : STATUS_RUNTIME;
}
int retro_trainer_generation_adapter_rows_info(retro_trainer * trainer, retro_adapter_rows_info * out_info) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_adapter_rows_info(g, out_info) : STATUS_RUNTIME;
}

// Reasoning budget (retro_lora_train.h:1680-1688, 2622-2627): -1 lets the model decide, N >= 0 forces the block's end
// tag after N reasoning tokens. The reference reads the tags out of the model's chat template; this library renders
// no templates, so the caller's template layer hands the tags over as token ids first (the extension below) and a
// budget without tags is refused with the reference's own message for a template without a reasoning block.
int retro_engine_set_reasoning_budget(retro_engine * engine, int32_t budget) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        return e ? e->set_reasoning_budget(budget) : STATUS_RUNTIME;
    });
}
int retro_trainer_set_reasoning_budget(retro_trainer * trainer, int32_t budget) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_engine_set_reasoning_budget(g, budget) : STATUS_RUNTIME;
}
int retro_b200_engine_set_reasoning_tags(retro_engine * engine, const int32_t * start, size_t n_start, const int32_t * const * end_tags,
                                         const size_t * n_end, size_t n_end_tags, size_t n_prompt_tail) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (n_end_tags && (!end_tags || !n_end)) {
            set_error("end_tags and n_end are required");
            return STATUS_RUNTIME;
        }
        return e->set_reasoning_tags(start, n_start, end_tags, n_end, n_end_tags, n_prompt_tail);
    });
}
int retro_b200_trainer_set_reasoning_tags(retro_trainer * trainer, const int32_t * start, size_t n_start, const int32_t * const * end_tags,
                                          const size_t * n_end, size_t n_end_tags, size_t n_prompt_tail) {
    retro_engine * g = generation_of(trainer);
    return g ? retro_b200_engine_set_reasoning_tags(g, start, n_start, end_tags, n_end, n_end_tags, n_prompt_tail) : STATUS_RUNTIME;
}

// ---- extensions -----------------------------------------------------------------------------

// Host logic only: runs one request's budget machine - primed with the end of `prompt`, then fed the tokens a
// sampler drew - and returns what the step would emit: out_tokens[i] and whether the budget forced it.
// `incomplete` lists token ids whose text stops inside a UTF-8 sequence.
int retro_b200_reasoning_check(const int32_t * start, size_t n_start, const int32_t * const * end_tags, const size_t * n_end, size_t n_end_tags,
                               int32_t budget, size_t n_prompt_tail, const int32_t * prompt, size_t n_prompt, const int32_t * incomplete,
                               size_t n_incomplete, const int32_t * sampled, size_t n_sampled, int32_t * out_tokens, uint8_t * out_forced) {
    return boundary([&]() -> int {
        if ((n_sampled && (!sampled || !out_tokens || !out_forced)) || (n_end_tags && (!end_tags || !n_end))) {
            set_error("reasoning_check: bad arguments");
            return STATUS_INVALID_ARGUMENT;
        }
        ReasoningPlan plan;
        if (n_start) plan.starts.emplace_back(start, start + n_start);
        for (size_t e = 0; e < n_end_tags; ++e)
            if (n_end[e]) plan.ends.emplace_back(end_tags[e], end_tags[e] + n_end[e]);
        if (!plan.ends.empty()) plan.forced = plan.ends.front();
        plan.budget = budget;
        plan.n_prompt_tail = n_prompt_tail;
        plan.active = budget >= 0 && !plan.starts.empty() && !plan.ends.empty();
        const std::vector<int32_t> partial(incomplete, incomplete + (incomplete ? n_incomplete : 0));
        BudgetMachine machine(&plan, [&](int32_t token) { return std::find(partial.begin(), partial.end(), token) == partial.end(); });
        machine.prime(prompt, prompt ? n_prompt : 0);
        for (size_t i = 0; i < n_sampled; ++i) {
            bool forced = false;
            out_tokens[i] = machine.next(sampled[i], forced);
            out_forced[i] = forced ? 1 : 0;
        }
        return STATUS_OK;
    });
}

int retro_b200_synth_gguf(const char * path, const char * spec, uint64_t * out_bytes) {
    return boundary([&]() -> int {
        if (is_blank(path)) {
            set_error("path is required");
            return STATUS_INVALID_ARGUMENT;
        }
        const uint64_t n = synth_gguf(path, spec);
        if (out_bytes) *out_bytes = n;
        return STATUS_OK;
    });
}

int retro_b200_quantize_row(uint32_t ggml_type, const float * values, size_t n, uint8_t * out, size_t n_out, size_t * out_bytes) {
    return boundary([&]() -> int {
        if (!values || !out) {
            set_error("values and out are required");
            return STATUS_INVALID_ARGUMENT;
        }
        const size_t need = row_bytes(ggml_type, n);
        if (need == 0) {
            set_error("unsupported type or partial block");
            return STATUS_INVALID_ARGUMENT;
        }
        if (n_out < need) {
            set_error("the output buffer is too small");
            return STATUS_BUFFER_TOO_SMALL;
        }
        const size_t written = quantize_row(ggml_type, values, n, out);
        if (written == 0) {
            set_error("unsupported type");
            return STATUS_INVALID_ARGUMENT;
        }
        if (out_bytes) *out_bytes = written;
        return STATUS_OK;
    });
}

int retro_b200_engine_last_pack(retro_engine * engine, size_t * n_tokens, size_t * n_out, int32_t * tok_slot, int32_t * tok_pos,
                                int32_t * tok_row, int32_t * tok_cell, int32_t * out_index, int32_t * cu_rows, size_t capacity) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (n_tokens) *n_tokens = e->last_T;
        if (n_out) *n_out = e->last_S;
        if (capacity < e->last_T || capacity < e->last_R + 1) {
            if (tok_slot || tok_pos || tok_row || tok_cell || out_index || cu_rows) {
                set_error("the map buffers are too small");
                return STATUS_BUFFER_TOO_SMALL;
            }
            return STATUS_OK;
        }
        auto fetch = [&](int32_t * dst, const int32_t * src, size_t n) {
            if (dst && n) RB_CUDA(cudaMemcpy(dst, src, n * 4, cudaMemcpyDeviceToHost));
        };
        fetch(tok_slot, e->maps.tok_slot, e->last_T);
        fetch(tok_pos, e->maps.tok_pos, e->last_T);
        fetch(tok_row, e->maps.tok_row, e->last_T);
        fetch(tok_cell, e->maps.tok_cell, e->last_T);
        fetch(out_index, e->maps.out_index, e->last_S);
        fetch(cu_rows, e->maps.cu_rows, e->last_R + 1);
        return STATUS_OK;
    });
}

int retro_b200_engine_last_logits(retro_engine * engine, size_t index, float * out, size_t n_vocab) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out) {
            if (e) set_error("out is required");
            return STATUS_RUNTIME;
        }
        if (index >= e->last_S || n_vocab < e->model->hp.vocab) {
            set_error("no such logits row in the last step");
            return STATUS_INVALID_ARGUMENT;
        }
        RB_CUDA(cudaMemcpy(out, e->logits.ptr + index * (size_t)e->model->hp.vocab, (size_t)e->model->hp.vocab * 4, cudaMemcpyDeviceToHost));
        return STATUS_OK;
    });
}

int retro_b200_engine_last_routes(retro_engine * engine, int32_t * out, size_t n_max, size_t * out_count) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        const size_t n = (size_t)e->model->hp.n_layer * e->last_T * e->model->hp.n_expert_used;
        if (out_count) *out_count = n;
        if (out && n) {
            if (n_max < n) {
                set_error("the route buffer is too small");
                return STATUS_BUFFER_TOO_SMALL;
            }
            RB_CUDA(cudaMemcpy(out, e->route_ids.ptr, n * 4, cudaMemcpyDeviceToHost));
        }
        return STATUS_OK;
    });
}

int retro_b200_engine_block_table(retro_engine * engine, int32_t slot, int32_t * out_blocks, size_t n_max, size_t * out_count,
                                  uint32_t * out_block_tokens) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (slot < 0 || slot >= (int32_t)e->config.n_seq_max) {
            set_error("slot is outside the context's sequence range");
            return STATUS_INVALID_ARGUMENT;
        }
        const KvSlot & s = e->kv->slot(slot);
        if (out_block_tokens) *out_block_tokens = e->kv->block_tokens();
        const size_t n = s.empty() ? 0 : (size_t)s.pos_max / e->kv->block_tokens() + 1;
        if (out_count) *out_count = n;
        if (out_blocks && n) {
            if (n_max < n) {
                set_error("the block buffer is too small");
                return STATUS_BUFFER_TOO_SMALL;
            }
            // read the device copy: it is what the kernels resolve positions through
            RB_CUDA(cudaMemcpy(out_blocks, e->kv_block_table_device() + (size_t)slot * e->kv->max_blocks(), n * 4, cudaMemcpyDeviceToHost));
            for (size_t i = 0; i < n; ++i) if (s.blocks[i] < 0) out_blocks[i] = -1;
        }
        return STATUS_OK;
    });
}

int retro_b200_engine_blocks(retro_engine * engine, uint64_t * out_used, uint64_t * out_total) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (out_used) *out_used = e->kv->blocks_used();
        if (out_total) *out_total = e->kv->n_blocks();
        return STATUS_OK;
    });
}

int retro_b200_engine_last_step_stats(retro_engine * engine, float * out_ms, uint64_t * out_launches) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (out_ms) *out_ms = e->last_ms;
        if (out_launches) *out_launches = e->last_launches;
        return STATUS_OK;
    });
}

int retro_b200_engine_graph_stats(retro_engine * engine, uint64_t * out_replays, uint64_t * out_cached) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        e->graph_stats(out_replays, out_cached);
        return STATUS_OK;
    });
}

namespace {
int invalid(const std::string & message) {
    set_error(message);
    return STATUS_INVALID_ARGUMENT;
}
} // namespace

int retro_b200_recode_mxfp4_as_q8_0(const void * mxfp4, size_t n_blocks, void * out_q8_0, int * out_recoded) {
    return boundary([&]() -> int {
        if (!mxfp4 || !out_q8_0 || !out_recoded) return invalid("retro_b200_recode_mxfp4_as_q8_0: null argument");
        std::vector<uint8_t> out;
        *out_recoded = mxfp4_to_q8_0(mxfp4, n_blocks * 17, out) ? 1 : 0;
        if (*out_recoded) std::memcpy(out_q8_0, out.data(), out.size());
        return STATUS_OK;
    });
}

int retro_b200_engine_expert_storage(retro_engine * engine, int layer, uint32_t * out_types_3) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (!out_types_3 || layer < 0 || layer >= (int)e->model->hp.n_layer || e->model->hp.n_expert == 0)
            return invalid("retro_b200_engine_expert_storage: not a layer of a mixture-of-experts model");
        const LayerWeights & lw = e->model->layers[layer];
        out_types_3[0] = lw.gate_exps.type;
        out_types_3[1] = lw.up_exps.type;
        out_types_3[2] = lw.down_exps.type;
        return STATUS_OK;
    });
}

int retro_b200_nccl_unique_id(void * out_id_128) {
    return boundary([&]() -> int {
        if (!out_id_128) return invalid("retro_b200_nccl_unique_id: null buffer");
        const int status = nccl_api().GetUniqueId(out_id_128);
        if (status != 0) throw std::runtime_error(std::string("NCCL: ") + nccl_api().GetErrorString(status));
        return STATUS_OK;
    });
}

int retro_b200_engine_ep_init(retro_engine * engine, int rank, int world, const void * unique_id_128) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        try {
            e->ep_init(rank, world, unique_id_128);
        } catch (const std::invalid_argument & err) {
            return invalid(err.what());
        }
        return STATUS_OK;
    });
}

int retro_b200_engine_ep_idle_step(retro_engine * engine) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        try {
            e->ep_idle_step();
        } catch (const std::invalid_argument & err) {
            return invalid(err.what());
        }
        return STATUS_OK;
    });
}

int retro_b200_ep_plan(const int32_t * all_offsets, int world, int rank, int n_expert, int32_t * send_begin, int32_t * send_count, int32_t * recv_begin,
                       int32_t * recv_count, int32_t * offsets, int32_t * sorted, int32_t sorted_capacity, int32_t * out_n_recv) {
    return boundary([&]() -> int {
        if (!all_offsets || world < 1 || rank < 0 || rank >= world || n_expert < 1 || n_expert % world != 0 || !send_begin || !send_count ||
            !recv_begin || !recv_count || !offsets || !out_n_recv)
            return invalid("retro_b200_ep_plan: bad arguments (the expert count must be a multiple of the world size)");
        EpPlan plan;
        ep_make_plan(all_offsets, world, rank, n_expert, plan);
        *out_n_recv = plan.n_recv;
        if (plan.n_recv > sorted_capacity || (plan.n_recv > 0 && !sorted)) {
            set_error("retro_b200_ep_plan: the sorted buffer is too small");
            return STATUS_BUFFER_TOO_SMALL;
        }
        std::copy(plan.send_begin.begin(), plan.send_begin.end(), send_begin);
        std::copy(plan.send_count.begin(), plan.send_count.end(), send_count);
        std::copy(plan.recv_begin.begin(), plan.recv_begin.end(), recv_begin);
        std::copy(plan.recv_count.begin(), plan.recv_count.end(), recv_count);
        std::copy(plan.offsets.begin(), plan.offsets.end(), offsets);
        std::copy(plan.sorted.begin(), plan.sorted.end(), sorted);
        return STATUS_OK;
    });
}

int retro_b200_checked_build(void) {
#ifdef RETRO_B200_CHECKED
    return 1;
#else
    return 0;
#endif
}

int retro_b200_engine_check_word(retro_engine * engine, int32_t out_word_4[4]) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e || !out_word_4) {
            if (e) set_error("out_word_4 is required");
            return STATUS_RUNTIME;
        }
        for (int i = 0; i < 4; ++i) out_word_4[i] = e->last_check[i];
        return STATUS_OK;
    });
}

int retro_b200_engine_last_step_io(retro_engine * engine, uint64_t * out_h2d_bytes, uint64_t * out_d2h_bytes) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (out_h2d_bytes) *out_h2d_bytes = e->last_h2d_bytes;
        if (out_d2h_bytes) *out_d2h_bytes = e->last_d2h_bytes;
        return STATUS_OK;
    });
}

int retro_b200_engine_profile(retro_engine * engine, int enabled, int reset) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        e->prof_.enabled = enabled != 0;
        if (reset) e->prof_.reset();
        return STATUS_OK;
    });
}

int retro_b200_engine_profile_read(retro_engine * engine, double * out_ms, uint64_t * out_launches, size_t n_classes) {
    return boundary([&]() -> int {
        Engine * e = checked(engine);
        if (!e) return STATUS_RUNTIME;
        if (n_classes < K_CLASS_COUNT) {
            set_error("the profile buffers are too small");
            return STATUS_BUFFER_TOO_SMALL;
        }
        for (int i = 0; i < K_CLASS_COUNT; ++i) {
            if (out_ms) out_ms[i] = e->prof_.ms[i];
            if (out_launches) out_launches[i] = e->prof_.launches[i];
        }
        return STATUS_OK;
    });
}

} // extern "C"
