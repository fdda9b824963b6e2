// The step executor: validates a step plan exactly as the reference's runtime does
// (crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:2399-2516 - same order, same messages,
// all-or-nothing before anything is decoded), then runs the whole decode on the GPU: packing maps
// and block-table resolution, the transformer forward over the paged KV cache, and sampling.
// One host->device copy carries the plan in, one device->host copy carries the sampled rows out.

#include "engine.hpp"
#include "blocks.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <unordered_set>

namespace rb200 {

std::string & last_error() {
    thread_local std::string message;
    return message;
}

namespace {

uint64_t fnv1a(const void * data, size_t n, uint64_t h = 0xcbf29ce484222325ULL) {
    const uint8_t * p = static_cast<const uint8_t *>(data);
    for (size_t i = 0; i < n; ++i) {
        h ^= p[i];
        h *= 0x100000001b3ULL;
    }
    return h;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

} // namespace

// ---------------------------------------------------------------------------------------------
// Model load

// MXFP4 blocks (E8M0 byte + 16 bytes of nibbles; element i in the low nibble of byte i, element 16 + i in
// its high nibble) -> Q8_0 blocks (f16 d + 32 int8) of the same values: d = 2^(x - 128) is half the E8M0
// scale, the int8 is the doubled E2M1 value. False when a block's scale is outside what an f16 holds.
bool mxfp4_to_q8_0(const void * src, size_t bytes, std::vector<uint8_t> & out) {
    static const int8_t doubled[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
    const size_t n_blocks = bytes / 17;
    const uint8_t * in = static_cast<const uint8_t *>(src);
    bool ok = true;
#pragma omp parallel for reduction(&& : ok)
    for (long long b = 0; b < (long long)n_blocks; ++b) {
        const int e = (int)in[b * 17] - 128;
        if (e < -24 || e > 15) ok = false;
    }
    if (!ok) return false;
    out.resize(n_blocks * 34);
#pragma omp parallel for
    for (long long b = 0; b < (long long)n_blocks; ++b) {
        const uint8_t * blk = in + b * 17;
        uint8_t * dst = out.data() + b * 34;
        const int e = (int)blk[0] - 128;
        // f16 bits of 2^e: normal for e >= -14, else the subnormal with mantissa bit e + 24
        const uint16_t d = e >= -14 ? (uint16_t)((e + 15) << 10) : (uint16_t)(1u << (e + 24));
        dst[0] = (uint8_t)(d & 0xFF);
        dst[1] = (uint8_t)(d >> 8);
        for (int i = 0; i < 16; ++i) {
            dst[2 + i] = (uint8_t)doubled[blk[1 + i] & 0xF];
            dst[2 + 16 + i] = (uint8_t)doubled[blk[1 + i] >> 4];
        }
    }
    return true;
}

void Engine::load_model(const std::string & path) {
    if (const char * env = std::getenv("RB200_MOE")) moe_tensor_cores_ = std::string(env) != "rows";
    if (const char * env = std::getenv("RB200_LORA")) lora_tensor_cores_ = std::string(env) != "rows";
    if (const char * env = std::getenv("RB200_Q8_TC5")) q8_tc5_ = std::string(env) != "0";
    GgufFile file(path);
    model = std::make_unique<Model>();
    Model & m = *model;
    HParams & hp = m.hp;
    hp.arch = file.str("general.architecture");
    if (hp.arch != "llama" && hp.arch != "qwen2" && hp.arch != "olmoe") {
        throw std::runtime_error("failed to load model GGUF: architecture '" + hp.arch + "' is not served by this backend");
    }
    const std::string a = hp.arch;
    hp.neox = a != "llama";
    hp.n_layer = file.u32(a + ".block_count", 0);
    hp.d = file.u32(a + ".embedding_length", 0);
    hp.n_head = file.u32(a + ".attention.head_count", 0);
    hp.n_head_kv = file.u32(a + ".attention.head_count_kv", hp.n_head);
    hp.ff = file.u32(a + ".feed_forward_length", 0);
    if (!hp.n_layer || !hp.d || !hp.n_head || !hp.n_head_kv || !hp.ff) throw std::runtime_error("failed to load model GGUF: missing hyper-parameters");
    hp.head_dim = file.u32(a + ".attention.key_length", hp.d / hp.n_head);
    hp.n_rot = file.u32(a + ".rope.dimension_count", hp.head_dim);
    hp.eps = file.f32(a + ".attention.layer_norm_rms_epsilon", 1e-5f);
    hp.rope_base = file.f32(a + ".rope.freq_base", 10000.f);
    hp.n_expert = file.u32(a + ".expert_count", 0);
    hp.n_expert_used = file.u32(a + ".expert_used_count", 0);
    if (hp.head_dim > 256 || hp.head_dim % 8 != 0) throw std::runtime_error("failed to load model GGUF: unsupported head size");
    if (hp.n_expert > 256) throw std::runtime_error("failed to load model GGUF: more than 256 experts");

    auto upload = [&](const void * src, size_t bytes) -> uint8_t * {
        void * p = nullptr;
        RB_CUDA(cudaMalloc(&p, align_up(bytes, 256)));
        m.allocations.push_back(p);
        RB_CUDA(cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice));
        m.weight_bytes += bytes;
        return static_cast<uint8_t *>(p);
    };
    auto need = [&](const std::string & name) -> const GgufTensor & {
        const GgufTensor * t = file.find(name);
        if (!t) throw std::runtime_error("failed to load model GGUF: missing tensor " + name);
        return *t;
    };
    // the host-side check the matrix' tcgen05 kernel asks for (see WeightView::tc5_exact)
    auto tc5_check = [&](const GgufTensor & t, uint64_t n_in) {
        if (t.type == GGML_Q4_K) return n_in % 256 == 0 && q4k_min_fold_ok(t.data, t.n_bytes / 144);
        if (t.type == GGML_Q8_0) return n_in % 64 == 0 && q8_0_products_fit_f16(t.data, t.n_bytes / 34);
        return false;
    };
    auto view_of = [&](const GgufTensor & t, const uint8_t * dev, uint64_t rows, bool tc5_exact) {
        WeightView w;
        w.tc5_exact = tc5_exact;
        w.data = dev;
        w.type = t.type;
        w.n_in = (uint32_t)t.ne[0];
        w.n_out = (uint32_t)rows;
        w.row_bytes = (uint32_t)row_bytes(t.type, t.ne[0]);
        const bool wants_tiled = t.ne.size() == 2 && w.n_in % 256 == 0 &&
                                 ((t.type == GGML_Q4_K && rows >= 128) || (t.type == GGML_Q8_0 && rows >= 16));
        // A blocking copy from pageable host memory may return while its last piece is still on its way
        // to the device; the regrouping kernels run on another stream, so wait for the device first.
        if (wants_tiled) RB_CUDA(cudaDeviceSynchronize());
        if (t.type == GGML_Q4_K && t.ne.size() == 2 && w.n_in % 256 == 0 && rows >= 128) {
            // second copy regrouped for the tcgen05 kernel's coalesced weight stream
            void * tiled = nullptr;
            const size_t bytes = q4k_tiled_bytes(w.n_out, w.n_in);
            RB_CUDA(cudaMalloc(&tiled, bytes));
            m.allocations.push_back(tiled);
            launch_q4k_retile(dev, w.n_out, w.n_in, w.row_bytes, static_cast<uint8_t *>(tiled), stream);
            w.tiled = static_cast<const uint8_t *>(tiled);
            m.tiled_bytes += bytes;
        } else if (t.type == GGML_Q8_0 && t.ne.size() == 2 && w.n_in % 256 == 0 && rows >= 16) {
            // second copy in MMA fragment order for the decode streaming kernel
            void * tiled = nullptr;
            const size_t bytes = q8_0_tiled_bytes(w.n_out, w.n_in);
            RB_CUDA(cudaMalloc(&tiled, bytes));
            m.allocations.push_back(tiled);
            launch_q8_0_retile(dev, w.n_out, w.n_in, w.row_bytes, static_cast<uint8_t *>(tiled), stream);
            w.tiled = static_cast<const uint8_t *>(tiled);
            m.tiled_bytes += bytes;
        }
        return w;
    };
    auto matrix = [&](const std::string & name, uint64_t n_in, uint64_t n_out) {
        const GgufTensor & t = need(name);
        if (t.ne.size() != 2 || t.ne[0] != n_in || t.ne[1] != n_out) throw std::runtime_error("failed to load model GGUF: unexpected shape of " + name);
        if (n_in % 8 != 0) throw std::runtime_error("failed to load model GGUF: row length of " + name + " is not a multiple of 8");
        return view_of(t, upload(t.data, t.n_bytes), n_out, tc5_check(t, n_in));
    };
    auto vector_f32 = [&](const std::string & name, uint64_t n, bool optional) -> const float * {
        const GgufTensor * t = file.find(name);
        if (!t) {
            if (optional) return nullptr;
            throw std::runtime_error("failed to load model GGUF: missing tensor " + name);
        }
        if (t->type != GGML_F32 || t->ne[0] != n) throw std::runtime_error("failed to load model GGUF: " + name + " must be F32 of the expected length");
        return reinterpret_cast<const float *>(upload(t->data, t->n_bytes));
    };
    // Several matrices with one row length and storage type, stacked row-wise into one allocation.
    auto fused = [&](const std::vector<std::string> & names, uint64_t n_in, const std::vector<uint64_t> & n_out, WeightView & out) -> bool {
        uint32_t type = need(names[0]).type;
        size_t total = 0;
        for (size_t i = 0; i < names.size(); ++i) {
            const GgufTensor & t = need(names[i]);
            if (t.type != type || t.ne.size() != 2 || t.ne[0] != n_in || t.ne[1] != n_out[i]) return false;
            total += t.n_bytes;
        }
        if (n_in % 8 != 0) return false;
        void * p = nullptr;
        RB_CUDA(cudaMalloc(&p, align_up(total, 256)));
        m.allocations.push_back(p);
        size_t off = 0;
        uint64_t rows = 0;
        bool tc5_exact = true;
        for (size_t i = 0; i < names.size(); ++i) {
            const GgufTensor & t = need(names[i]);
            tc5_exact = tc5_exact && tc5_check(t, n_in);
            RB_CUDA(cudaMemcpy(static_cast<uint8_t *>(p) + off, t.data, t.n_bytes, cudaMemcpyHostToDevice));
            off += t.n_bytes;
            rows += n_out[i];
        }
        m.weight_bytes += total;
        out = view_of(need(names[0]), static_cast<uint8_t *>(p), rows, tc5_exact);
        return true;
    };

    const GgufTensor & embd = need("token_embd.weight");
    hp.vocab = (uint32_t)embd.ne[1];
    if (embd.ne[0] != hp.d) throw std::runtime_error("failed to load model GGUF: token_embd width differs from embedding_length");
    m.token_embd = view_of(embd, upload(embd.data, embd.n_bytes), hp.vocab, tc5_check(embd, hp.d));

    const uint64_t dq = hp.dq(), dkv = hp.dkv();
    m.layers.resize(hp.n_layer);
    for (uint32_t l = 0; l < hp.n_layer; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        LayerWeights & lw = m.layers[l];
        lw.attn_norm = vector_f32(p + "attn_norm.weight", hp.d, false);
        if (!fused({p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"}, hp.d, {dq, dkv, dkv}, lw.wqkv)) {
            lw.wq = matrix(p + "attn_q.weight", hp.d, dq);
            lw.wk = matrix(p + "attn_k.weight", hp.d, dkv);
            lw.wv = matrix(p + "attn_v.weight", hp.d, dkv);
        }
        if (file.find(p + "attn_q.bias")) {
            std::vector<float> b(dq + 2 * dkv);
            const GgufTensor & bq = need(p + "attn_q.bias");
            const GgufTensor & bk = need(p + "attn_k.bias");
            const GgufTensor & bv = need(p + "attn_v.bias");
            if (bq.type != GGML_F32 || bk.type != GGML_F32 || bv.type != GGML_F32 || bq.ne[0] != dq || bk.ne[0] != dkv || bv.ne[0] != dkv) {
                throw std::runtime_error("failed to load model GGUF: attention biases must be F32 of the projection width");
            }
            std::memcpy(b.data(), bq.data, dq * 4);
            std::memcpy(b.data() + dq, bk.data, dkv * 4);
            std::memcpy(b.data() + dq + dkv, bv.data, dkv * 4);
            lw.bqkv = reinterpret_cast<const float *>(upload(b.data(), b.size() * 4));
        }
        lw.q_norm = vector_f32(p + "attn_q_norm.weight", dq, true);
        lw.k_norm = vector_f32(p + "attn_k_norm.weight", dkv, true);
        lw.wo = matrix(p + "attn_output.weight", dq, hp.d);
        lw.ffn_norm = vector_f32(p + "ffn_norm.weight", hp.d, false);
        if (hp.n_expert == 0) {
            if (!fused({p + "ffn_gate.weight", p + "ffn_up.weight"}, hp.d, {hp.ff, hp.ff}, lw.wgu)) {
                lw.wgate = matrix(p + "ffn_gate.weight", hp.d, hp.ff);
                lw.wup = matrix(p + "ffn_up.weight", hp.d, hp.ff);
            }
            lw.wdown = matrix(p + "ffn_down.weight", hp.ff, hp.d);
        } else {
            lw.router = matrix(p + "ffn_gate_inp.weight", hp.d, hp.n_expert);
            if (lw.router.type != GGML_F32) throw std::runtime_error("failed to load model GGUF: the router must be F32");
            // MXFP4 banks whose every weight is an f16 (E8M0 bytes 104..128) and whose rows are whole 64-column groups are
            // held ONLY in the tiled layout of the grouped tcgen05 GEMM: the format's own 17 bytes per 32 weights.
            bool mxfp4_direct = moe_tensor_cores_ && tensor_maps_available() && hp.d % 64 == 0 && hp.ff % 64 == 0;
            for (const char * stem : {"ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"}) {
                const GgufTensor & t = need(p + stem);
                mxfp4_direct = mxfp4_direct && t.type == GGML_MXFP4 && t.ne.size() == 3 && mxfp4_scales_are_f16(t.data, t.n_bytes / 17);
            }
            auto bank = [&](const std::string & name, uint64_t n_in, uint64_t n_out, WeightView & w, uint64_t & stride) {
                const GgufTensor & t = need(name);
                if (t.ne.size() != 3 || t.ne[0] != n_in || t.ne[1] != n_out || t.ne[2] != hp.n_expert || n_in % 8 != 0) {
                    throw std::runtime_error("failed to load model GGUF: unexpected shape of " + name);
                }
                if (mxfp4_direct) {
                    void * raw = nullptr, * tiled = nullptr;
                    RB_CUDA(cudaMalloc(&raw, align_up(t.n_bytes, 256)));
                    RB_CUDA(cudaMemcpy(raw, t.data, t.n_bytes, cudaMemcpyHostToDevice));
                    const size_t bytes = mxfp4_tiled_bytes(hp.n_expert, (uint32_t)n_out, (uint32_t)n_in);
                    RB_CUDA(cudaMalloc(&tiled, bytes));
                    m.allocations.push_back(tiled);
                    RB_CUDA(cudaDeviceSynchronize());       // the blocking upload has reached the device
                    launch_mxfp4_retile(static_cast<const uint8_t *>(raw), hp.n_expert, (uint32_t)n_out, (uint32_t)n_in, static_cast<uint8_t *>(tiled), stream);
                    RB_CUDA(cudaStreamSynchronize(stream));
                    RB_CUDA(cudaFree(raw));
                    w = WeightView{};
                    w.type = GGML_MXFP4;
                    w.n_in = (uint32_t)n_in;
                    w.n_out = (uint32_t)n_out;
                    w.row_bytes = (uint32_t)row_bytes(GGML_MXFP4, n_in);
                    w.tiled = static_cast<const uint8_t *>(tiled);
                    m.weight_bytes += bytes;
                    stride = 0;
                    return;
                }
                // MXFP4 experts whose block scales are powers of two an f16 holds are re-coded, exactly, as Q8_0
                // (the doubled E2M1 value as the int8, half the E8M0 scale as d): the tensor-core Q8_0 GEMM
                // then serves the experts. Twice the bytes per weight, an order of magnitude faster than the
                // CUDA-core row kernel.
                std::vector<uint8_t> recoded;
                if (t.type == GGML_MXFP4 && moe_tensor_cores_ && n_in % 64 == 0 && mxfp4_to_q8_0(t.data, t.n_bytes, recoded)) {
                    w.data = upload(recoded.data(), recoded.size());
                    w.type = GGML_Q8_0;
                    w.n_in = (uint32_t)n_in;
                    w.n_out = (uint32_t)n_out;
                    w.row_bytes = (uint32_t)row_bytes(GGML_Q8_0, n_in);
                } else {
                    w = view_of(t, upload(t.data, t.n_bytes), n_out, false);
                }
                stride = (uint64_t)w.row_bytes * n_out;
            };
            bank(p + "ffn_gate_exps.weight", hp.d, hp.ff, lw.gate_exps, lw.gate_stride);
            bank(p + "ffn_up_exps.weight", hp.d, hp.ff, lw.up_exps, lw.up_stride);
            bank(p + "ffn_down_exps.weight", hp.ff, hp.d, lw.down_exps, lw.down_stride);
            // the inventory entry of each bank, as the file holds it (retro_experts.cpp:86-131: role = the
            // name's stem without "ffn_" and "_exps")
            const char * roles[3] = {"gate", "up", "down"};
            const WeightView * views[3] = {&lw.gate_exps, &lw.up_exps, &lw.down_exps};
            for (int b = 0; b < 3; ++b) {
                const GgufTensor & t = need(p + "ffn_" + roles[b] + "_exps.weight");
                retro_expert_bank_desc desc{};
                desc.layer = l;
                std::snprintf(desc.role, sizeof desc.role, "%s", roles[b]);
                std::snprintf(desc.tensor.name, sizeof desc.tensor.name, "%s", t.name.c_str());
                desc.tensor.n_elements = 1;
                for (int i = 0; i < 4; ++i) {
                    desc.tensor.ne[i] = i < (int)t.ne.size() ? (int64_t)t.ne[i] : 1;
                    desc.tensor.n_elements *= (uint64_t)desc.tensor.ne[i];
                }
                desc.tensor.n_bytes = t.n_bytes;
                desc.tensor.storage_id = reinterpret_cast<uint64_t>(views[b]->data);
                const char * type = t.type == GGML_F32 ? "F32" : t.type == GGML_F16 ? "F16" : t.type == GGML_BF16 ? "BF16" : t.type == GGML_Q8_0 ? "Q8_0"
                                    : t.type == GGML_Q4_K ? "Q4_K" : t.type == GGML_MXFP4 ? "MXFP4" : "unknown";
                std::snprintf(desc.tensor.type_name, sizeof desc.tensor.type_name, "%s", type);
                m.expert_banks.push_back(desc);
            }
        }
    }
    m.output_norm = vector_f32("output_norm.weight", hp.d, false);
    if (file.find("output.weight")) {
        m.output = matrix("output.weight", hp.d, hp.vocab);
    } else {
        m.output = m.token_embd;   // tied head
    }
    m.output_bias = vector_f32("output.bias", hp.vocab, true);

    std::vector<float> inv(hp.n_rot / 2);
    for (uint32_t i = 0; i < hp.n_rot / 2; ++i) inv[i] = (float)std::pow((double)hp.rope_base, -2.0 * i / hp.n_rot);
    m.inv_freq.ensure(inv.size());
    RB_CUDA(cudaMemcpy(m.inv_freq.ptr, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice));

    if (const auto * toks = file.str_array("tokenizer.ggml.tokens")) m.vocab_tokens = *toks;
    if (const auto * types = file.i32_array("tokenizer.ggml.token_type")) m.vocab_types = *types;
    m.eos = (int32_t)file.u32("tokenizer.ggml.eos_token_id", 2);
    m.bos = (int32_t)file.u32("tokenizer.ggml.bos_token_id", 1);
    m.add_bos = file.u32("tokenizer.ggml.add_bos_token", 1) != 0;
    std::sort(m.expert_banks.begin(), m.expert_banks.end(),
              [](const retro_expert_bank_desc & a, const retro_expert_bank_desc & b) { return std::strcmp(a.tensor.name, b.tensor.name) < 0; });
    // End of generation is more than EOS: the end-of-turn and end-of-message ids the file names, and the control
    // tokens chat formats end a turn with (a Llama-3 chat turn ends with <|eot_id|>, not with EOS).
    m.eog.assign(hp.vocab, 0);
    auto mark = [&](int64_t id) { if (id >= 0 && id < (int64_t)hp.vocab) m.eog[(size_t)id] = 1; };
    mark(m.eos);
    for (const char * key : {"tokenizer.ggml.eot_token_id", "tokenizer.ggml.eom_token_id"}) {
        const uint32_t id = file.u32(key, UINT32_MAX);
        if (id != UINT32_MAX) mark(id);
    }
    static const char * const end_of_turn_pieces[] = {"<|eot_id|>", "<|im_end|>", "<|end|>", "<|eom_id|>", "<end_of_turn>", "<|endoftext|>",
                                                       "<|end_of_text|>", "<|return|>", "<|call|>", "<EOT>"};
    for (size_t i = 0; i < m.vocab_tokens.size() && i < hp.vocab; ++i) {
        const int32_t type = i < m.vocab_types.size() ? m.vocab_types[i] : 3;
        if (type != 3 && type != 4) continue;       // control or user-defined pieces only
        for (const char * piece : end_of_turn_pieces)
            if (m.vocab_tokens[i] == piece) m.eog[i] = 1;
    }

    // every blocking upload above has reached the device before any stream's kernel reads the weights
    RB_CUDA(cudaDeviceSynchronize());
    // fingerprint = FNV-1a(path || u64 file size), as the reference keys its prefix caches
    uint64_t h = fnv1a(path.data(), path.size());
    const uint64_t size = file.file_size();
    fingerprint = fnv1a(&size, sizeof size, h);
}

std::string Model::piece(int32_t token, bool unparse_special) const {
    if (token < 0 || (size_t)token >= vocab_tokens.size()) return "";
    const std::string & t = vocab_tokens[token];
    const int32_t type = (size_t)token < vocab_types.size() ? vocab_types[token] : 1;
    if (type == 6 && t.size() == 6 && t[0] == '<' && t[1] == '0' && t[2] == 'x') return std::string(1, (char)std::stoi(t.substr(3, 2), nullptr, 16));
    if (type == 3 || type == 2) return unparse_special ? t : "";
    std::string out;
    for (size_t i = 0; i < t.size();) {
        if (i + 2 < t.size() && (uint8_t)t[i] == 0xE2 && (uint8_t)t[i + 1] == 0x96 && (uint8_t)t[i + 2] == 0x81) {
            out.push_back(' ');
            i += 3;
        } else {
            out.push_back(t[i++]);
        }
    }
    return out;
}

// ---------------------------------------------------------------------------------------------

Engine::Engine(const std::string & path, const retro_engine_config & cfg) : config(cfg), model_path(path) {
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
        throw std::runtime_error("device=gpu requested but no GPU backend is available; this library has no CPU path");
    }
    RB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    RB_CUDA(cudaStreamCreateWithFlags(&side_stream_, cudaStreamNonBlocking));
    RB_CUDA(cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming));
    RB_CUDA(cudaEventCreateWithFlags(&ev_join_, cudaEventDisableTiming));
    if (const char * env = std::getenv("RB200_ATTN_OVERLAP")) attn_overlap_ = std::string(env) != "0";
    if (const char * env = std::getenv("RB200_KV_Q8_NATIVE")) kv_q8_native_ = std::string(env) != "0";
    RB_CUDA(cudaEventCreate(&ev_begin_));
    RB_CUDA(cudaEventCreate(&ev_end_));
    load_model(path);
    const HParams & hp = model->hp;
    n_ctx_seq = config.kv_unified ? config.n_ctx : config.n_ctx / config.n_seq_max;
    if (n_ctx_seq == 0) throw std::runtime_error("failed to create the engine context: n_ctx is smaller than n_seq_max on a partitioned pool");

    const uint32_t n_blocks = (config.n_ctx + kBlockTokens - 1) / kBlockTokens + config.n_seq_max;
    const uint32_t max_blocks = (n_ctx_seq + kBlockTokens - 1) / kBlockTokens;
    kv = std::make_unique<KvManager>(config.n_seq_max, n_blocks, kBlockTokens, max_blocks);
    kv_layer_stride_ = (uint64_t)n_blocks * hp.n_head_kv * kBlockTokens * hp.head_dim;
    kv_storage_ = config.kv_dtype == RETRO_ENGINE_KV_DTYPE_Q8_0 ? KV_Q8_0 : config.kv_dtype == RETRO_ENGINE_KV_DTYPE_Q4_0 ? KV_Q4_0 : KV_F16;
    if (config.kv_dtype == RETRO_ENGINE_KV_DTYPE_F32)
        throw std::runtime_error("this backend stores the KV cache as F16, Q8_0 or Q4_0: engine kv_dtype F32 is not supported");
    if (kv_storage_ != KV_F16) {
        // The pool holds ggml's quantised rows; the attention kernels read one layer at a time from an f16 scratch
        // with the pool's block numbering, which kv_dequant fills for the step's sequences.
        if (hp.head_dim % 32 != 0) throw std::runtime_error("a quantized engine kv_dtype needs a head dimension that is a multiple of 32");
        kv_q_layer_stride_ = (uint64_t)n_blocks * hp.n_head_kv * kBlockTokens * kv_row_bytes(kv_storage_, (int)hp.head_dim);
        kq_.ensure(kv_q_layer_stride_ * hp.n_layer);
        vq_.ensure(kv_q_layer_stride_ * hp.n_layer);
        RB_CUDA(cudaMemsetAsync(kq_.ptr, 0, kq_.count, stream));
        RB_CUDA(cudaMemsetAsync(vq_.ptr, 0, vq_.count, stream));
    }
    const uint64_t f16_layers = kv_storage_ == KV_F16 ? hp.n_layer : 1;
    kcache_.ensure(kv_layer_stride_ * f16_layers);
    vcache_.ensure(kv_layer_stride_ * f16_layers);
    // Cells past a sequence's end in its last block are read (and masked) by the attention kernels:
    // a masked probability of zero times a leftover NaN bit pattern would still be NaN.
    RB_CUDA(cudaMemsetAsync(kcache_.ptr, 0, kcache_.count * sizeof(__half), stream));
    RB_CUDA(cudaMemsetAsync(vcache_.ptr, 0, vcache_.count * sizeof(__half), stream));
    block_table_.ensure((size_t)config.n_seq_max * max_blocks);
    RB_CUDA(cudaMemsetAsync(block_table_.ptr, 0, block_table_.count * 4, stream));

    const size_t T = config.n_batch;
    maps_store_.ensure(T * 9 + 3 * (T + 1) + 8);
    int32_t * p = maps_store_.ptr;
    maps.cu_rows = p; p += T + 1;
    maps.out_rank = p; p += T + 1;
    maps.tok_slot = p; p += T;
    maps.tok_pos = p; p += T;
    maps.tok_row = p; p += T;
    maps.tok_cell = p; p += T;
    maps.tok_adapter = p; p += T;
    maps.tok_pos_min = p; p += T;
    maps.out_index = p; p += T;
    maps.tile_rank = p; p += T + 1;
    p += (reinterpret_cast<uintptr_t>(p) & 7) ? 1 : 0;     // int2 alignment
    maps.attn_items = reinterpret_cast<int2 *>(p);
    attn_mma_ = attention_mma_supported((int)hp.n_head, (int)hp.n_head_kv, (int)hp.head_dim, (int)kBlockTokens);
    if (const char * env = std::getenv("RB200_ATTENTION")) attn_mma_ = attn_mma_ && std::string(env) != "ref";
    attn_tile_tokens_ = attn_mma_ ? kAttentionTileRows / (int)(hp.n_head / hp.n_head_kv) : 64;
    // prefill tiles on tcgen05 with TMA-staged K/V (RB200_ATTN_TC5=0: the mma.sync tile kernel)
    attn_tc5_ = attn_mma_;
    if (const char * env = std::getenv("RB200_ATTN_TC5")) attn_tc5_ = attn_tc5_ && std::string(env) != "0";
    if (attn_tc5_) {
        attention_maps_encode(attn_maps_, kcache_.ptr, vcache_.ptr, (int)hp.head_dim, f16_layers * (kv_layer_stride_ / hp.head_dim));
        attn_tc5_ = attention_tc5_supported((int)hp.n_head, (int)hp.n_head_kv, (int)hp.head_dim, (int)kBlockTokens, attn_maps_);
    }

    x_.ensure(T * hp.d);
    xn_.ensure(T * hp.d);
    qkv_.ensure(T * (hp.dq() + 2 * hp.dkv()));
    att_.ensure(T * hp.dq());
    xn_split_.ensure(T, hp.d);
    att_split_.ensure(T, hp.dq());
    if (hp.n_expert == 0) hff_split_.ensure(T, hp.ff);
    if (const char * env = std::getenv("RB200_GEMM")) {
        if (std::string(env) == "mma") tc5_min_tokens = 1 << 30;     // keep the mma.sync kernels for every token count
    }
    {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm_, cudaDevAttrMultiProcessorCount, dev);
        if (const char * env = std::getenv("RB200_GEMM")) stream_gemm_ = std::string(env) != "rows";
        if (const char * env = std::getenv("RB200_GRAPHS")) graphs_enabled_ = std::string(env) != "0";
        if (const char * env = std::getenv("RB200_FUSED_FINISH")) fused_finish_ = std::string(env) != "0";
        if (const char * env = std::getenv("RB200_ATTENTION")) attn_decode8_ = std::string(env) != "decode16";
    }
    device_error_.ensure(1);
    RB_CUDA(cudaMemsetAsync(device_error_.ptr, 0, sizeof(int), stream));
#ifdef RETRO_B200_CHECKED
    check_word_.ensure(4);
    RB_CUDA(cudaMemsetAsync(check_word_.ptr, 0, 4 * sizeof(int), stream));
    maps.check = check_word_.ptr;
#endif
    maps.n_slots = (int32_t)config.n_seq_max;
    maps.n_blocks = (int32_t)n_blocks;
    if (const char * env = std::getenv("RB200_MMA_MIN_TOKENS")) mma_min_tokens = std::atoi(env);
    if (hp.n_expert == 0) {
        gu_.ensure(T * 2 * hp.ff);
        hff_.ensure(T * hp.ff);
    } else {
        const size_t P = T * hp.n_expert_used;
        router_logits_.ensure(T * hp.n_expert);
        moe_ids_.ensure(P);
        moe_offsets_.ensure(hp.n_expert + 1);
        moe_sorted_.ensure(P);
        moe_w_.ensure(P);
        pair_gu_.ensure(P * 2 * hp.ff);
        pair_h_.ensure(P * hp.ff);
        pair_y_.ensure(P * hp.d);
        route_ids.ensure((size_t)hp.n_layer * P);
        route_counts.assign(hp.n_layer, std::vector<uint32_t>(hp.n_expert, 0));
    }
    RB_CUDA(cudaStreamSynchronize(stream));
}

Engine::~Engine() {
    if (stream) cudaStreamSynchronize(stream);
    if (ep_comm_) {
        try { nccl_api().CommDestroy(ep_comm_); } catch (...) {}
    }
    if (h_ep_offsets_) cudaFreeHost(h_ep_offsets_);
    if (h_stage_) cudaFreeHost(h_stage_);
    if (h_result_) cudaFreeHost(h_result_);
    if (ev_fork_) cudaEventDestroy(ev_fork_);
    if (ev_join_) cudaEventDestroy(ev_join_);
    if (side_stream_) cudaStreamDestroy(side_stream_);
    if (ev_begin_) cudaEventDestroy(ev_begin_);
    if (ev_end_) cudaEventDestroy(ev_end_);
    if (stream) cudaStreamDestroy(stream);
}

KvLayout Engine::kv_layout() const {
    KvLayout l;
    l.k = kcache_.ptr;
    l.v = vcache_.ptr;
    l.layer_stride = kv_storage_ == KV_F16 ? kv_layer_stride_ : 0;
    l.kq = kq_.ptr;
    l.vq = vq_.ptr;
    l.q_layer_stride = kv_q_layer_stride_;
    l.storage = kv_storage_;
    l.q_row_bytes = kv_storage_ == KV_F16 ? 0 : kv_row_bytes(kv_storage_, (int)model->hp.head_dim);
    l.n_head_kv = (int32_t)model->hp.n_head_kv;
    l.head_dim = (int32_t)model->hp.head_dim;
    l.block_tokens = (int32_t)kBlockTokens;
    l.block_table = block_table_.ptr;
    l.max_blocks = (int32_t)kv->max_blocks();
    l.n_blocks = (int32_t)kv->n_blocks();
    l.check = check_word_.ptr;
    return l;
}

// Applies queued block-table patches and copy-on-write block copies outside a step
// (sequence operations issued between steps).
void Engine::flush_kv_updates() {
    std::vector<int32_t> & patches = kv->patches();
    std::vector<int32_t> & copies = kv->copies();
    if (patches.empty() && copies.empty()) return;
    const size_t n = patches.size() + copies.size();
    d_aux_.ensure(n);
    std::vector<int32_t> host(patches);
    host.insert(host.end(), copies.begin(), copies.end());
    RB_CUDA(cudaMemcpyAsync(d_aux_.ptr, host.data(), n * 4, cudaMemcpyHostToDevice, stream));
    launch_block_table_patch(block_table_.ptr, d_aux_.ptr, (int)(patches.size() / 2), stream, (int)block_table_.count, (int)kv->n_blocks(), check_word_.ptr);
    launch_kv_block_copy(kv_layout(), (int)model->hp.n_layer, d_aux_.ptr + patches.size(), (int)(copies.size() / 2), stream);
    RB_CUDA(cudaStreamSynchronize(stream));
    patches.clear();
    copies.clear();
}

// 9..16 tokens: a second pass of the weight stream costs more than the tcgen05 kernel when that one
// can cut the reduction into splits (matrices with few 128-row tiles), measured on the 8B shapes.
bool Engine::tc5_split_preferred(const WeightView & w, int T, const SplitAct * xs) const {
    return xs && T > 8 && T <= kStreamMaxTokens && tc5_min_tokens <= kStreamMaxTokens && gemm_q4k_tc5_supported(w, *xs) &&
           gemm_q4k_tc5_splits(w.n_out, w.n_in, T, n_sm_) > 1;
}

// Returns whether `tail` (the row-wise step that consumes y) was done by the GEMM's own finish kernel.
bool Engine::linear(const WeightView & w, const float * x, int ldx, int T, float * y, int ldy, const float * bias, const float * residual,
                    int ldr, const SplitAct * xs, const FinishTail * tail) {
    bool tail_done = false;
    prof_.begin(K_GEMM, stream);
    if (xs && stream_gemm_ && T <= kStreamMaxTokens && !tc5_split_preferred(w, T, xs) &&
               (gemm_q4k_stream_supported(w, *xs, std::min(T, 8)) || gemm_q8_0_stream_supported(w, *xs, std::min(T, 8)))) {
        // at most 8 tokens per pass of the weight stream; up to 16 tokens two passes still beat the tensor-core kernels
        stream_scratch_.ensure(gemm_q4k_stream_scratch_floats(w.n_out, w.n_in));
        tail_done = tail && fused_finish_ && finish_tail_supported(*tail, (int)w.n_out, y, ldy, bias, residual, ldr);
        for (int t0 = 0; t0 < T; t0 += 8) {
            const int n = std::min(8, T - t0);
            SplitAct part = *xs;
            part.hi += (size_t)t0 * xs->ld;
            part.lo += (size_t)t0 * xs->ld;
            part.sum_hi += (size_t)t0 * (xs->ld / 32);
            part.sum_lo += (size_t)t0 * (xs->ld / 32);
            const float * res = residual ? residual + (size_t)t0 * ldr : nullptr;
            FinishTail part_tail;
            RopeStoreArgs part_rope;
            if (tail_done) {
                part_tail = *tail;
                if (part_tail.rope) {
                    part_rope = *part_tail.rope;
                    part_rope.tok_pos += t0;
                    part_rope.tok_cell += t0;
                    part_tail.rope = &part_rope;
                }
                if (part_tail.out) part_tail.out += (size_t)t0 * part_tail.ld_out;
                if (part_tail.split.hi) {
                    part_tail.split.hi += (size_t)t0 * part_tail.split.ld;
                    part_tail.split.lo += (size_t)t0 * part_tail.split.ld;
                    part_tail.split.sum_hi += (size_t)t0 * (part_tail.split.ld / 32);
                    part_tail.split.sum_lo += (size_t)t0 * (part_tail.split.ld / 32);
                }
            }
            const FinishTail * pass_tail = tail_done ? &part_tail : nullptr;
            if (w.type == GGML_Q4_K)
                launch_gemm_q4k_stream(w, part, n, y + (size_t)t0 * ldy, ldy, bias, res, ldr, stream_scratch_.ptr, n_sm_, device_error_.ptr, stream,
                                       pass_tail);
            else
                launch_gemm_q8_0_stream(w, part, n, y + (size_t)t0 * ldy, ldy, bias, res, ldr, stream_scratch_.ptr, n_sm_, device_error_.ptr, stream,
                                        pass_tail);
            last_launches += 2;
        }
        --last_launches;        // the common tail below counts one
    } else if (xs && (T > tc5_min_tokens || tc5_split_preferred(w, T, xs)) && gemm_q4k_tc5_supported(w, *xs)) {
        const size_t need = gemm_q4k_tc5_scratch_floats(w.n_out, w.n_in, T, n_sm_);
        if (need) stream_scratch_.ensure(need);
        tail_done = need && tail && fused_finish_ && finish_tail_supported(*tail, (int)w.n_out, y, ldy, bias, residual, ldr);
        launch_gemm_q4k_tc5(w, *xs, T, y, ldy, bias, residual, ldr, device_error_.ptr, need ? stream_scratch_.ptr : nullptr, stream_scratch_.count, n_sm_,
                            stream, tail_done ? tail : nullptr);
        if (need) ++last_launches;
    } else if (xs && T > mma_min_tokens && gemm_q4k_exact_supported(w, *xs)) {
        launch_gemm_q4k_exact(w, *xs, T, y, ldy, bias, residual, ldr, stream);
    } else if (xs && T > mma_min_tokens && q8_tc5_ && gemm_q8_0_tc5_supported(w, *xs)) {
        launch_gemm_q8_0_tc5(w, *xs, T, y, ldy, bias, residual, ldr, device_error_.ptr, n_sm_, stream);
} else if (xs && T > mma_min_tokens && gemm_q8_0_exact_supported(w, *xs)) {
        launch_gemm_q8_0_exact(w, *xs, T, y, ldy, bias, residual, ldr, stream);
    } else {
        launch_gemm_rows(w, x, ldx, T, y, ldy, bias, residual, ldr, stream);
    }
    prof_.end(K_GEMM, 1, stream);
    ++last_launches;
    return tail_done;
}

// Runs one step's device work: eagerly, or as a replayed / freshly captured CUDA graph.
void Engine::run_step_work(const std::vector<uint64_t> & sig, const std::function<void()> & issue) {
    // (under expert parallelism every MoE layer synchronises with the host for its exchange plan: eager only)
    const bool graphable = graphs_enabled_ && !prof_.enabled && !ep_comm_;
    if (graph_epoch_ != g_alloc_epoch.load()) {       // some buffer moved: every captured pointer is stale
        for (auto & e : graphs_) if (e.second.exec) cudaGraphExecDestroy(e.second.exec);
        graphs_.clear();
        graph_epoch_ = g_alloc_epoch.load();
    }
    GraphEntry * entry = nullptr;
    if (graphable) {
        uint64_t key = 1469598103934665603ull;
        for (uint64_t v : sig) key = (key ^ v) * 1099511628211ull;
        auto it = graphs_.find(key);
        if (it != graphs_.end() && it->second.sig != sig) {       // a collision: forget the old entry
            if (it->second.exec) cudaGraphExecDestroy(it->second.exec);
            graphs_.erase(it);
            it = graphs_.end();
        }
        if (it == graphs_.end()) {
            if (graphs_.size() >= 64) {
                for (auto & e : graphs_) if (e.second.exec) cudaGraphExecDestroy(e.second.exec);
                graphs_.clear();
            }
            it = graphs_.emplace(key, GraphEntry{sig, nullptr, 0, 0}).first;
        }
        entry = &it->second;
    }
    RB_CUDA(cudaEventRecord(ev_begin_, stream));
    if (entry && entry->exec) {
        RB_CUDA(cudaGraphLaunch(entry->exec, stream));
        last_launches = entry->launches;
        ++graph_replays_;
    } else if (entry && entry->seen >= 1 && !entry->failed) {
        // second occurrence: capture, instantiate, launch
        const uint64_t epoch_before = g_alloc_epoch.load();
        cudaGraph_t graph = nullptr;
        bool ok = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if (ok) {
            try {
                issue();
            } catch (...) {
                cudaStreamEndCapture(stream, &graph);
                if (graph) cudaGraphDestroy(graph);
                cudaGetLastError();
                entry->failed = true;
                throw;
            }
            ok = cudaStreamEndCapture(stream, &graph) == cudaSuccess && graph != nullptr;
        }
        if (ok && epoch_before == g_alloc_epoch.load()) ok = cudaGraphInstantiate(&entry->exec, graph, 0) == cudaSuccess;
        else ok = false;
        if (graph) cudaGraphDestroy(graph);
        if (ok) {
            entry->launches = last_launches;
            RB_CUDA(cudaGraphLaunch(entry->exec, stream));
        } else {
            cudaGetLastError();
            entry->exec = nullptr;
            entry->failed = true;
            issue();            // nothing ran during the failed capture
        }
    } else {
        issue();
        if (entry) ++entry->seen;
    }
    RB_CUDA(cudaEventRecord(ev_end_, stream));
}

// Whether linear() will read the split form of the activations for this weight and token count
// (then the f32 copy of the activations need not be written at all).
bool Engine::linear_reads_split(const WeightView & w, int ldx, int T, const SplitAct * xs) const {
    if (!xs) return false;
    if (stream_gemm_ && T <= kStreamMaxTokens &&
        (gemm_q4k_stream_supported(w, *xs, std::min(T, 8)) || gemm_q8_0_stream_supported(w, *xs, std::min(T, 8))))
        return true;
    if ((T > tc5_min_tokens || tc5_split_preferred(w, T, xs)) && gemm_q4k_tc5_supported(w, *xs)) return true;
    return T > mma_min_tokens && (gemm_q4k_exact_supported(w, *xs) || gemm_q8_0_exact_supported(w, *xs) || (q8_tc5_ && gemm_q8_0_tc5_supported(w, *xs)));
}

void Engine::lora(const std::string & target, const float * x, int ldx, int T, float * y, int ldy) {
    lora_group({target}, {0}, x, ldx, T, y, ldy);
}

// The adapters' deltas of up to three targets that read the same rows x: y[:, offsets[i] + ...] += scale B_i (A_i x).
void Engine::lora_group(const std::vector<std::string> & targets, const std::vector<int> & y_offsets, const float * x, int ldx, int T, float * y, int ldy) {
    if (!cur_any_adapter_) return;
    LoraGroup group;
    std::vector<LoraTarget *> present;
    std::vector<int> offsets_present;
    for (size_t i = 0; i < targets.size(); ++i) {
        auto it = lora_targets_.find(targets[i]);
        if (it == lora_targets_.end() || !it->second->present) continue;
        present.push_back(it->second.get());
        offsets_present.push_back(y_offsets[i]);
    }
    if (present.empty()) return;
    const uint32_t n_in = present[0]->n_in;
    bool grouped = lora_tensor_cores_ && adapters_.size() <= 1024 && present.size() <= (size_t)kLoraTcMaxTargets &&
                   lora_tc_supported((int)r_max_, (int)n_in, present[0]->a.ptr, x, ldx);
    for (LoraTarget * t : present) grouped = grouped && t->n_in == n_in && (uintptr_t)t->a.ptr % 16 == 0;
    prof_.begin(K_LORA, stream);
    if (grouped) {
        for (size_t i = 0; i < present.size(); ++i) {
            group.a[i] = present[i]->a.ptr;
            group.b[i] = present[i]->b.ptr;
            group.n_out[i] = (int)present[i]->n_out;
            group.y_offset[i] = offsets_present[i];
        }
        group.n = (int)present.size();
        launch_lora_tc(group, lora_scales_.ptr, (int)r_max_, (int)n_in, (int)adapters_.size(), lora_offsets_.ptr, lora_sorted_.ptr, x, ldx, T,
                       lora_tmp_.ptr, y, ldy, stream);
        prof_.end(K_LORA, 2, stream);
        last_launches += 2;
        return;
    }
    for (size_t i = 0; i < present.size(); ++i) {
        LoraTarget & t = *present[i];
        if (t.n_in % 4 == 0 && ldx % 4 == 0 && adapters_.size() <= 1024)
            launch_lora_shrink_grouped(t.a.ptr, (int)r_max_, (int)t.n_in, (int)adapters_.size(), lora_offsets_.ptr, lora_sorted_.ptr, x, ldx, lora_tmp_.ptr,
                                       stream);
        else
            launch_lora_shrink(t.a.ptr, (int)r_max_, (int)t.n_in, cur_tok_adapter_, x, ldx, T, lora_tmp_.ptr, stream);
        launch_lora_expand(t.b.ptr, (int)r_max_, (int)t.n_out, lora_scales_.ptr, cur_tok_adapter_, lora_tmp_.ptr, T, y + offsets_present[i], ldy, stream);
        last_launches += 2;
    }
    prof_.end(K_LORA, 2 * (uint32_t)present.size(), stream);
}

// ---------------------------------------------------------------------------------------------
// Expert FFNs on the tensor cores

bool Engine::moe_experts_on_tensor_cores(const LayerWeights & lw) const {
    const HParams & hp = model->hp;
    if (lw.gate_exps.type == GGML_MXFP4 && lw.gate_exps.tiled) return true;        // the tiled MXFP4 banks of the grouped tcgen05 GEMM
    return moe_tensor_cores_ && lw.gate_exps.type == GGML_Q8_0 && lw.up_exps.type == GGML_Q8_0 && lw.down_exps.type == GGML_Q8_0 &&
           hp.d % 64 == 0 && hp.ff % 64 == 0;
}

// The experts' SwiGLU FFN over n (row, expert) pairs whose expert-sorted order is `gather`: pair i reads row
// gather[i] / gather_div of `rows` and its result goes to row gather[i] of y_out. d_offsets (device,
// n_expert + 1) delimits each expert's pairs. The exact Q8_0 tensor-core GEMM runs in its grouped form, one
// launch for all experts with fixed token tiles: an element's arithmetic does not depend on how many pairs
// its expert has, which keeps results independent of the grouping (and of the expert-parallel world size).
void Engine::moe_experts_tc(const LayerWeights & lw, const float * rows, int ld_rows, const int32_t * gather, int gather_div,
                            const int32_t * d_offsets, int n, float * y_out, int ld_out) {
    const HParams & hp = model->hp;
    const int E = (int)hp.n_expert, d = (int)hp.d, ff = (int)hp.ff;
    if (n <= 0) return;
    if ((size_t)n > moe_split_rows_) {
        moe_split_rows_ = (size_t)n + (size_t)n / 2;
        moe_x_split_.ensure(moe_split_rows_, d);
        moe_h_split_.ensure(moe_split_rows_, ff);
    }
    moe_gu_s_.ensure((size_t)n * 2 * ff);
    moe_y_s_.ensure((size_t)n * d);
    // the pairs' activation rows, gathered into expert order and split in one pass
    launch_split_prep(rows, ld_rows, d, n, moe_x_split_.view, stream, gather, gather_div);
    if (gemm_mxfp4_tc5_supported(lw.gate_exps, moe_x_split_.view) && gemm_mxfp4_tc5_supported(lw.down_exps, moe_h_split_.view)) {
        launch_gemm_mxfp4_tc5_grouped(lw.gate_exps, E, d_offsets, moe_x_split_.view, n, moe_gu_s_.ptr, 2 * ff, device_error_.ptr, stream);
        launch_gemm_mxfp4_tc5_grouped(lw.up_exps, E, d_offsets, moe_x_split_.view, n, moe_gu_s_.ptr + ff, 2 * ff, device_error_.ptr, stream);
        launch_swiglu(moe_gu_s_.ptr, 2 * ff, ff, n, nullptr, ff, stream, &moe_h_split_.view);
        launch_gemm_mxfp4_tc5_grouped(lw.down_exps, E, d_offsets, moe_h_split_.view, n, moe_y_s_.ptr, d, device_error_.ptr, stream);
    } else {
        if (!lw.gate_exps.data) throw std::runtime_error("the expert banks are held for the tcgen05 kernel only, but its activation descriptors are unavailable");
        launch_gemm_q8_0_exact_grouped(lw.gate_exps, lw.gate_stride, E, d_offsets, moe_x_split_.view, n, moe_gu_s_.ptr, 2 * ff, stream);
        launch_gemm_q8_0_exact_grouped(lw.up_exps, lw.up_stride, E, d_offsets, moe_x_split_.view, n, moe_gu_s_.ptr + ff, 2 * ff, stream);
        launch_swiglu(moe_gu_s_.ptr, 2 * ff, ff, n, nullptr, ff, stream, &moe_h_split_.view);
        launch_gemm_q8_0_exact_grouped(lw.down_exps, lw.down_stride, E, d_offsets, moe_h_split_.view, n, moe_y_s_.ptr, d, stream);
    }
    launch_ep_scatter_rows(moe_y_s_.ptr, gather, n, d, y_out, ld_out, stream);
    last_launches += 6;
}

// ---------------------------------------------------------------------------------------------
// Expert parallelism

#define RB_NCCL(call)                                                                                          \
    do {                                                                                                       \
        const int rb_nccl_status = (call);                                                                     \
        if (rb_nccl_status != 0) throw std::runtime_error(std::string("NCCL: ") + nccl_api().GetErrorString(rb_nccl_status)); \
    } while (0)

void Engine::ep_init(int rank, int world, const void * unique_id_128) {
    const HParams & hp = model->hp;
    if (hp.n_expert == 0) throw std::invalid_argument("expert parallelism needs a mixture-of-experts model");
    if (ep_comm_) throw std::invalid_argument("expert parallelism is already initialised for this engine");
    if (world < 1 || rank < 0 || rank >= world || !unique_id_128) throw std::invalid_argument("expert parallelism: bad rank / world size");
    if (hp.n_expert % (uint32_t)world != 0) throw std::invalid_argument("expert parallelism: the expert count is not a multiple of the world size");
    const NcclApi & nccl = nccl_api();
    NcclId128 id;
    std::memcpy(id.bytes, unique_id_128, sizeof(id.bytes));
    RB_NCCL(nccl.CommInitRank(&ep_comm_, world, id, rank));
    ep_rank_ = rank;
    ep_world_ = world;
    ep_all_offsets_.ensure((size_t)world * (hp.n_expert + 1));
    ep_offsets_l_.ensure(hp.n_expert + 1);
    ep_flags_.ensure((size_t)world + 1);
    RB_CUDA(cudaMallocHost(reinterpret_cast<void **>(&h_ep_offsets_), ((size_t)world * (hp.n_expert + 1) + world + 1) * sizeof(int32_t)));
    if (world > 1) ep_keep_local_experts();
}

// From here on this rank serves experts [rank * E / world, (rank + 1) * E / world) only: every bank is replaced by
// a copy of that range and the full bank is freed, so the experts' footprint is divided by the world size like
// their weight stream. The views keep indexing by GLOBAL expert id: their base address is moved back by the
// bytes of the experts in front of the range. An expert outside the range never has rows on this rank (the
// exchange plan sends every pair to its expert's owner), and every grouped kernel returns on an empty row range
// before it forms a weight address.
void Engine::ep_keep_local_experts() {
    Model & m = *model;
    const uint32_t per = m.hp.n_expert / (uint32_t)ep_world_, first = (uint32_t)ep_rank_ * per;
    RB_CUDA(cudaStreamSynchronize(stream));
    auto keep = [&](WeightView & w, uint64_t stride) {
        const bool tiled_only = w.type == GGML_MXFP4 && w.tiled && !w.data;
        const uint8_t * old = tiled_only ? w.tiled : w.data;
        const size_t per_expert = tiled_only ? mxfp4_tiled_bytes(1, w.n_out, w.n_in) : (size_t)stride;
        if (!old || per_expert == 0) return;
        void * local = nullptr;
        RB_CUDA(cudaMalloc(&local, align_up(per * per_expert, 256)));
        RB_CUDA(cudaMemcpy(local, old + (size_t)first * per_expert, per * per_expert, cudaMemcpyDeviceToDevice));
        auto it = std::find(m.allocations.begin(), m.allocations.end(), (void *)old);
        if (it != m.allocations.end()) {
            RB_CUDA(cudaFree(*it));
            *it = local;
        } else {
            m.allocations.push_back(local);
        }
        const uint8_t * biased = reinterpret_cast<const uint8_t *>(reinterpret_cast<uintptr_t>(local) - (uintptr_t)first * per_expert);
        (tiled_only ? w.tiled : w.data) = biased;
        m.weight_bytes -= (size_t)(m.hp.n_expert - per) * per_expert;
        ep_local_bank_bytes_ += per * per_expert;
    };
    for (LayerWeights & lw : m.layers) {
        keep(lw.gate_exps, lw.gate_stride);
        keep(lw.up_exps, lw.up_stride);
        keep(lw.down_exps, lw.down_stride);
    }
}

// Rows [begin[p], begin[p] + count[p]) of `send` go to rank p, rows from rank p land at recv_begin[p]. Both
// sides derive the counts from the same all-gathered offsets, so every send has its receive.
void Engine::ep_exchange(const float * send, const std::vector<int32_t> & send_begin, const std::vector<int32_t> & send_count, float * recv,
                         const std::vector<int32_t> & recv_begin, const std::vector<int32_t> & recv_count, int d) {
    const NcclApi & nccl = nccl_api();
    if (send_count[ep_rank_] > 0) {
        RB_CUDA(cudaMemcpyAsync(recv + (size_t)recv_begin[ep_rank_] * d, send + (size_t)send_begin[ep_rank_] * d, (size_t)send_count[ep_rank_] * d * 4,
                                cudaMemcpyDeviceToDevice, stream));
    }
    RB_NCCL(nccl.GroupStart());
    for (int p = 0; p < ep_world_; ++p) {
        if (p == ep_rank_) continue;
        if (send_count[p] > 0) RB_NCCL(nccl.Send(send + (size_t)send_begin[p] * d, (size_t)send_count[p] * d, kNcclFloat32, p, ep_comm_, stream));
        if (recv_count[p] > 0) RB_NCCL(nccl.Recv(recv + (size_t)recv_begin[p] * d, (size_t)recv_count[p] * d, kNcclFloat32, p, ep_comm_, stream));
    }
    RB_NCCL(nccl.GroupEnd());
}

// One MoE layer under expert parallelism. On entry: xn_ holds the T normalised tokens, moe_ids_ / moe_w_ the
// routing, moe_offsets_ / moe_sorted_ the pairs grouped by expert (T = 0: this rank only serves the others).
void Engine::ep_moe_layer(const LayerWeights & lw, int T) {
    const HParams & hp = model->hp;
    const NcclApi & nccl = nccl_api();
    const int E = (int)hp.n_expert, K = (int)hp.n_expert_used, P = T * K, d = (int)hp.d, ff = (int)hp.ff;
    if (P == 0) RB_CUDA(cudaMemsetAsync(moe_offsets_.ptr, 0, (size_t)(E + 1) * 4, stream));
    RB_NCCL(nccl.AllGather(moe_offsets_.ptr, ep_all_offsets_.ptr, (size_t)(E + 1), kNcclInt32, ep_comm_, stream));
    RB_CUDA(cudaMemcpyAsync(h_ep_offsets_, ep_all_offsets_.ptr, (size_t)ep_world_ * (E + 1) * 4, cudaMemcpyDeviceToHost, stream));
    RB_CUDA(cudaStreamSynchronize(stream));
    // the plan outlives this call: its vectors are the source of host-to-device copies, and the next
    // rewrite happens only after the next layer's stream synchronisation above
    EpPlan & plan = ep_plan_;
    ep_make_plan(h_ep_offsets_, ep_world_, ep_rank_, E, plan);
    const int n_recv = plan.n_recv;

    ep_send_.ensure((size_t)std::max(P, 1) * d);
    ep_back_.ensure((size_t)std::max(P, 1) * d);
    ep_recv_.ensure((size_t)std::max(n_recv, 1) * d);
    ep_gu_.ensure((size_t)std::max(n_recv, 1) * 2 * ff);
    ep_h_.ensure((size_t)std::max(n_recv, 1) * ff);
    ep_y_.ensure((size_t)std::max(n_recv, 1) * d);
    ep_sorted_l_.ensure((size_t)std::max(n_recv, 1));

    launch_ep_gather_rows(xn_.ptr, d, moe_sorted_.ptr, K, P, d, ep_send_.ptr, stream);
    ep_exchange(ep_send_.ptr, plan.send_begin, plan.send_count, ep_recv_.ptr, plan.recv_begin, plan.recv_count, d);
    if (n_recv > 0 && moe_experts_on_tensor_cores(lw)) {
        RB_CUDA(cudaMemcpyAsync(ep_offsets_l_.ptr, plan.offsets.data(), (size_t)(E + 1) * 4, cudaMemcpyHostToDevice, stream));
        RB_CUDA(cudaMemcpyAsync(ep_sorted_l_.ptr, plan.sorted.data(), (size_t)n_recv * 4, cudaMemcpyHostToDevice, stream));
        moe_experts_tc(lw, ep_recv_.ptr, d, ep_sorted_l_.ptr, 1, ep_offsets_l_.ptr, n_recv, ep_y_.ptr, d);
    } else if (n_recv > 0) {
        RB_CUDA(cudaMemcpyAsync(ep_offsets_l_.ptr, plan.offsets.data(), (size_t)(E + 1) * 4, cudaMemcpyHostToDevice, stream));
        RB_CUDA(cudaMemcpyAsync(ep_sorted_l_.ptr, plan.sorted.data(), (size_t)n_recv * 4, cudaMemcpyHostToDevice, stream));
        launch_moe_gemm_grouped(lw.gate_exps, lw.gate_stride, E, ep_offsets_l_.ptr, ep_sorted_l_.ptr, ep_recv_.ptr, d, 1, ep_gu_.ptr, 2 * ff, stream);
        launch_moe_gemm_grouped(lw.up_exps, lw.up_stride, E, ep_offsets_l_.ptr, ep_sorted_l_.ptr, ep_recv_.ptr, d, 1, ep_gu_.ptr + ff, 2 * ff, stream);
        launch_swiglu(ep_gu_.ptr, 2 * ff, ff, n_recv, ep_h_.ptr, ff, stream);
        launch_moe_gemm_grouped(lw.down_exps, lw.down_stride, E, ep_offsets_l_.ptr, ep_sorted_l_.ptr, ep_h_.ptr, ff, 1, ep_y_.ptr, d, stream);
    }
    // the results travel back along the same ranges, in the order the rows were sent
    ep_exchange(ep_y_.ptr, plan.recv_begin, plan.recv_count, ep_back_.ptr, plan.send_begin, plan.send_count, d);
    if (P > 0) {
        launch_ep_scatter_rows(ep_back_.ptr, moe_sorted_.ptr, P, d, pair_y_.ptr, d, stream);
        launch_moe_combine(pair_y_.ptr, d, moe_ids_.ptr, moe_w_.ptr, K, d, T, x_.ptr, x_.ptr, stream);
    }
    last_launches += 8;
}

// Every step under expert parallelism opens with this exchange: each rank says whether its own plan passed
// validation and KV reservation, and the step runs only if all of them did. A rank whose plan was refused
// returns its ordinary error; the others undo their reservation and return a runtime error of their own.
// Without it a refused rank would leave its peers waiting in the first layer's exchange for a partner that
// never comes. True when every rank is ready.
bool Engine::ep_agree(bool ready) {
    const NcclApi & nccl = nccl_api();
    int32_t * h_flags = h_ep_offsets_ + (size_t)ep_world_ * (model->hp.n_expert + 1);
    h_flags[ep_world_] = ready ? 1 : 0;
    RB_CUDA(cudaMemcpyAsync(ep_flags_.ptr + ep_world_, h_flags + ep_world_, sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    RB_NCCL(nccl.AllGather(ep_flags_.ptr + ep_world_, ep_flags_.ptr, 1, kNcclInt32, ep_comm_, stream));
    RB_CUDA(cudaMemcpyAsync(h_flags, ep_flags_.ptr, (size_t)ep_world_ * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    RB_CUDA(cudaStreamSynchronize(stream));
    for (int r = 0; r < ep_world_; ++r)
        if (!h_flags[r]) return false;
    return true;
}

// A step of a rank that has no rows of its own: its experts still serve the other ranks' tokens.
void Engine::ep_idle_step() {
    if (!ep_comm_) throw std::invalid_argument("expert parallelism is not initialised for this engine");
    if (!ep_agree(true)) return;        // a peer refused its step: nobody exchanges anything
    for (uint32_t l = 0; l < model->hp.n_layer; ++l) ep_moe_layer(model->layers[l], 0);
    RB_CUDA(cudaStreamSynchronize(stream));
}

// ---------------------------------------------------------------------------------------------
// The step

namespace {

// The all-or-nothing checks of a step plan, reported before anything is decoded. Contract (the
// reference's runtime, retro_gen_core.cpp:1509-1590 and :2409-2516): rows are examined in order, each
// row's checks in the order of `check_row` below, the first failure decides the message, the status is
// -3. What is free is how the answer is found: a row is compared only with the earlier rows of ITS
// slot (kept per slot in arrival order, which also yields the earliest conflicting row the reference's
// pair scan would have met first) and request ids are looked up in a hash set.
class PlanChecker {
public:
    PlanChecker(int32_t n_slots, int32_t n_batch, int64_t ctx_seq, int32_t n_vocab, bool have_top_buffers, size_t top_stride)
        : n_slots_(n_slots), n_batch_(n_batch), ctx_seq_(ctx_seq), n_vocab_(n_vocab), have_top_buffers_(have_top_buffers), top_stride_(top_stride) {}

    size_t tokens = 0, sampling_rows = 0;

    // `per_row_adapter(id)`: whether a positive adapter id names a loaded per-row adapter.
    template <class AdapterLookup> bool check_row(const EffRow * rows, size_t r, AdapterLookup && per_row_adapter) {
        const EffRow & row = rows[r];
        const bool v2 = row.v2 != nullptr;
        const size_t needed = v2 ? offsetof(retro_step_row_v2, adapter) + sizeof(int32_t) : offsetof(retro_step_row, adapter) + sizeof(int32_t);
        if (row.struct_size < needed)
            return refuse(v2 ? "retro_step_row_v2.struct_size is too small for this build" : "retro_step_row.struct_size is too small for this build");
        if (!row.tokens || row.n == 0) return refuse("a step row requires at least one token");
        if (row.slot < 0 || row.slot >= n_slots_) return refuse("step row slot is outside the context's sequence range");
        if (row.adapter != 0 && row.adapter != RETRO_STEP_ADAPTER_BASE && !per_row_adapter(row.adapter))
            return refuse("step row adapter " + std::to_string(row.adapter) + " is not a loaded per-row adapter");
        const int64_t begin = row.pos0, end = begin + row.n;
        if (begin < 0 || end > ctx_seq_) return refuse("step row positions exceed the per-sequence context");
        std::vector<uint32_t> & earlier = rows_of_slot_[row.slot];
        for (uint32_t e : earlier) {
            const EffRow & other = rows[e];
            if (begin < (int64_t)other.pos0 + other.n && other.pos0 < end) return refuse("step rows overlap in the same sequence slot");
            if (row.adapter != other.adapter) return refuse("step rows of one sequence slot select different adapters");
        }
        earlier.push_back((uint32_t)r);
        if (!tokens_in_vocabulary(row.tokens, row.n)) return false;
        if (row.n > (uint32_t)n_batch_ || tokens + row.n > (size_t)n_batch_) return refuse("the step's tokens exceed the context's physical batch (n_batch)");
        tokens += row.n;
        if (row.n_top_logprobs > 0 && !have_top_buffers_) return refuse("top logprobs requested but the output buffers are missing");
        if (row.n_top_logprobs > top_stride_) return refuse("a step row's n_top_logprobs exceeds the output stride");
        if (row.sample) {
            if (row.request < 0) return refuse("a sampling step row requires a request id");
            if (v2 ? !sampling_v2_ok(*row.v2) : !sampling_v1_ok(row.v1)) return false;
            ++sampling_rows;
        }
        if (row.request >= 0 && !requests_.insert(row.request).second) return refuse("a request id appears twice in one step");
        return true;
    }

private:
    struct Rule {
        bool (*broken)(const retro_sampling_params_v2 &);
        const char * message;
    };

    static bool refuse(const std::string & message) {
        set_error(message);
        return false;
    }
    static bool positive_finite(float v) { return v > 0.0f && std::isfinite(v); }
    static bool unit_interval_open_low(float v) { return v > 0.0f && v <= 1.0f; }

    bool tokens_in_vocabulary(const int32_t * ids, size_t n) const {
        for (size_t i = 0; i < n; ++i) {
            if (ids[i] >= 0 && ids[i] < n_vocab_) continue;
            return refuse("token " + std::to_string(ids[i]) + " at index " + std::to_string(i) + " is outside the vocabulary of size " +
                          std::to_string(n_vocab_));
        }
        return true;
    }
    // v1 rows: only the distribution parameters take part (the caller owns stopping, so max_new_tokens is not read)
    static bool sampling_v1_ok(const retro_sampling_params & s) {
        if (!positive_finite(s.temperature)) return refuse("sampling temperature must be finite and greater than zero");
        if (!unit_interval_open_low(s.top_p)) return refuse("sampling top_p must be in (0, 1]");
        return true;
    }
    bool sampling_v2_ok(const retro_sampling_params_v2 & s) const {
        static const Rule rules[] = {
            {[](const retro_sampling_params_v2 & p) { return p.struct_size < sizeof(retro_sampling_params_v2); },
             "retro_sampling_params_v2.struct_size is too small for this build"},
            {[](const retro_sampling_params_v2 & p) { return !positive_finite(p.temperature); }, "sampling temperature must be finite and greater than zero"},
            {[](const retro_sampling_params_v2 & p) { return !unit_interval_open_low(p.top_p); }, "sampling top_p must be in (0, 1]"},
            {[](const retro_sampling_params_v2 & p) { return !positive_finite(p.repeat_penalty); }, "sampling repeat_penalty must be finite and greater than zero"},
            {[](const retro_sampling_params_v2 & p) { return !(p.min_p >= 0.0f && p.min_p <= 1.0f); }, "sampling min_p must be in [0, 1]"},
            {[](const retro_sampling_params_v2 & p) { return !std::isfinite(p.frequency_penalty); }, "sampling frequency_penalty must be finite"},
            {[](const retro_sampling_params_v2 & p) { return !std::isfinite(p.presence_penalty); }, "sampling presence_penalty must be finite"},
            {[](const retro_sampling_params_v2 & p) { return p.n_logit_bias > 4096; }, "sampling n_logit_bias must not exceed 4096"},
            {[](const retro_sampling_params_v2 & p) { return p.n_logit_bias > 0 && (!p.logit_bias_ids || !p.logit_bias_values); },
             "logit_bias ids and values are required when n_logit_bias is nonzero"},
        };
        for (const Rule & rule : rules)
            if (rule.broken(s)) return refuse(rule.message);
        if (s.n_logit_bias == 0) return true;
        if (!tokens_in_vocabulary(s.logit_bias_ids, s.n_logit_bias)) return false;
        for (uint32_t i = 0; i < s.n_logit_bias; ++i)
            if (!std::isfinite(s.logit_bias_values[i])) return refuse("logit_bias values must be finite");
        return true;
    }

    int32_t n_slots_, n_batch_;
    int64_t ctx_seq_;
    int32_t n_vocab_;
    bool have_top_buffers_;
    size_t top_stride_;
    std::unordered_map<int32_t, std::vector<uint32_t>> rows_of_slot_;
    std::unordered_set<int32_t> requests_;
};

} // namespace

int Engine::step(const EffRow * rows, size_t n_rows, OutRow * out_rows, int32_t * out_top_ids, float * out_top_logprobs, size_t n_top_stride) {
    const HParams & hp = model->hp;
    // Under expert parallelism a refused plan still takes part in the step's opening exchange (ep_agree), so that
    // the peers skip the step instead of waiting for this rank; the message set before it is kept.
    auto refused = [&](int status) {
        if (ep_comm_) {
            const std::string message = last_error();
            try { ep_agree(false); } catch (...) {}
            set_error(message);
        }
        return status;
    };
    if (!rows || n_rows == 0 || !out_rows) {
        set_error("step rows and output rows are required");
        return refused(STATUS_INVALID_ARGUMENT);
    }
    if (n_rows > (size_t)config.n_batch || (n_top_stride != 0 && n_rows > SIZE_MAX / n_top_stride)) {
        set_error("the step row count or output shape exceeds capacity");
        return refused(STATUS_INVALID_ARGUMENT);
    }
    PlanChecker plan((int32_t)config.n_seq_max, (int32_t)config.n_batch, (int64_t)n_ctx_seq, (int32_t)hp.vocab, out_top_ids && out_top_logprobs, n_top_stride);
    const auto per_row_adapter = [this](int32_t id) {
        const auto found = adapters_.find(id);
        return found != adapters_.end() && !found->second.serial;
    };
    for (size_t r = 0; r < n_rows; ++r)
        if (!plan.check_row(rows, r, per_row_adapter)) return refused(STATUS_INVALID_ARGUMENT);
    const size_t total = plan.tokens, n_sample = plan.sampling_rows;
    // Grammars are compiled before anything is decoded, once per request and text (retro_gen_core.cpp:2518-2537):
    // a request keeps its place in its grammar from step to step as long as its rows carry the same GBNF.
    std::vector<std::shared_ptr<const Grammar>> fresh_grammars(n_rows);
    bool any_grammar = false;
    for (size_t r = 0; r < n_rows; ++r) {
        if (!rows[r].sample || !rows[r].v2 || !rows[r].v2->grammar) continue;
        any_grammar = true;
        const std::string & gbnf = rows[r].v2->grammar->gbnf;
        const auto known = requests.find(rows[r].request);
        if (known != requests.end() && known->second.grammar && known->second.grammar->gbnf == gbnf) continue;
        try {
            fresh_grammars[r] = std::make_shared<const Grammar>(gbnf);
        } catch (const std::invalid_argument & err) {
            set_error(std::string("failed to compile the request's grammar (invalid GBNF): ") + err.what());
            return refused(STATUS_INVALID_ARGUMENT);
        }
    }

    // ---- KV reservation: all rows or none
    kv->begin();
    for (size_t r = 0; r < n_rows; ++r) {
        const KvManager::Reserve res = kv->reserve(rows[r].slot, rows[r].pos0, (int32_t)rows[r].n);
        if (res != KvManager::OK) {
            kv->rollback();
            if (res == KvManager::GAP) {
                set_error("a step row starts past the end of its slot's resident sequence: positions must extend the slot without a gap");
            } else {
                set_error("the KV cache is full: no free block for the step's tokens (query the extent with the seq_pos entry point)");
            }
            return refused(STATUS_RUNTIME);
        }
    }
    if (ep_comm_ && !ep_agree(true)) {
        kv->rollback();
        set_error("another rank of the expert-parallel group refused its step: this rank's step was skipped and nothing was decoded");
        return STATUS_RUNTIME;
    }
    kv->commit();

    // ---- stage the plan
    const size_t T = total, R = n_rows, S = n_sample;
    std::vector<int32_t> & patches = kv->patches();
    std::vector<int32_t> & copies = kv->copies();
    std::vector<SampleDesc> descs(S);
    std::vector<LogitEdit> edits;
    // grammar rows: one bit per token, staged with the plan (the mask depends on the grammar's state, not on the logits)
    const size_t mask_words = (hp.vocab + 31) / 32;
    std::vector<uint32_t> masks;
    std::vector<std::unique_ptr<GrammarState>> row_grammar(n_rows);     // the state a row samples under; installed on success
    bool grammar_dead_end = false;
    if (any_grammar && token_pieces_.empty()) {
        token_pieces_.resize(hp.vocab);
        for (uint32_t t = 0; t < hp.vocab; ++t) token_pieces_[t] = model->piece((int32_t)t, false);
    }
    // reasoning budget: every request's machine follows the engine's current plan, and until its first sampling
    // row collects the end of its prompt across chunks (retro_gen_core.cpp:2609-2645)
    if (reasoning_plan_.active || reasoning_seen_) {
        reasoning_seen_ = true;
        for (size_t r = 0; r < R; ++r) {
            const EffRow & row = rows[r];
            if (row.request < 0) continue;
            RequestState & req = requests[row.request];
            if (!req.plan || !(*req.plan == reasoning_plan_)) {
                req.plan = std::make_unique<ReasoningPlan>(reasoning_plan_);
                const Model * mdl = model.get();
                req.budget = BudgetMachine(req.plan.get(), [mdl](int32_t token) { return utf8_is_complete(mdl->piece(token, true)); });
                req.primed = false;
                req.prompt_tail.clear();
            }
            if (!reasoning_plan_.active || req.primed) continue;
            req.prompt_tail.insert(req.prompt_tail.end(), row.tokens, row.tokens + row.n);
            if (req.prompt_tail.size() > reasoning_plan_.n_prompt_tail)
                req.prompt_tail.erase(req.prompt_tail.begin(), req.prompt_tail.end() - (ptrdiff_t)reasoning_plan_.n_prompt_tail);
        }
    }
    bool forced_outside_grammar = false;
    size_t top_stride = 0;
    bool any_v2 = false;       // some row needs the working copy of the logits
    int n_greedy_fast = 0;
    {
        size_t s = 0;
        for (size_t r = 0; r < R; ++r) {
            const EffRow & row = rows[r];
            if (!row.sample) continue;
            RequestState & req = requests[row.request];
            if (!req.seeded) {
                req.seed = row.v2 ? row.v2->seed : row.v1.seed;
                req.seeded = true;
            }
            if (req.budget.active() && !req.primed) {
                req.budget.prime(req.prompt_tail.data(), req.prompt_tail.size());
                req.primed = true;
            }
            const int32_t forced_token = req.budget.pending();
            SampleDesc & d = descs[s++];
            std::memset(&d, 0, sizeof d);
            if (forced_token >= 0) d.pad[1] = (uint32_t)forced_token + 1;
            d.seed = req.seed;
            d.draw_lo = (uint32_t)req.draws;
            d.draw_hi = (uint32_t)(req.draws >> 32);
            d.n_top = std::min<uint32_t>(row.n_top_logprobs, (uint32_t)std::min<size_t>(n_top_stride, hp.vocab));
            top_stride = std::max<size_t>(top_stride, d.n_top);
            d.edit_begin = d.edit_end = (uint32_t)edits.size();
            if (row.v2) {
                const retro_sampling_params_v2 & p = *row.v2;
                d.temperature = p.temperature;
                d.top_p = p.top_p;
                d.top_k = p.top_k;
                d.min_p = p.min_p;
                d.flags = 1u | (row.want_logprob ? 2u : 0u);
                if (p.grammar) {
                    auto state = std::make_unique<GrammarState>();
                    if (fresh_grammars[r]) {
                        state->grammar = fresh_grammars[r];
                        state->gbnf = p.grammar->gbnf;
                        state->stacks = state->grammar->initial();
                    } else {
                        *state = *req.grammar;
                    }
                    d.pad[0] = (uint32_t)masks.size() + 1;       // word offset of this row's mask, plus one
                    masks.resize(masks.size() + mask_words, 0u);
                    uint32_t * bits = masks.data() + masks.size() - mask_words;
                    const GrammarState & g = *state;
                    bool any_allowed = false;
#pragma omp parallel for schedule(static) reduction(|| : any_allowed)
                    for (long long t = 0; t < (long long)hp.vocab; ++t) {
                        if (!g.allows(token_pieces_[t], model->is_eog((int32_t)t))) continue;
#pragma omp atomic
                        bits[t >> 5] |= 1u << (t & 31);
                        any_allowed = true;
                    }
                    grammar_dead_end = grammar_dead_end || !any_allowed;
                    if (forced_token >= 0 && !g.allows(token_pieces_[forced_token], model->is_eog(forced_token))) forced_outside_grammar = true;
                    row_grammar[r] = std::move(state);
                }
                // one merged edit per distinct id: summed bias, then the penalties of the window
                std::map<int32_t, LogitEdit> merged;
                for (uint32_t i = 0; i < p.n_logit_bias; ++i) {
                    LogitEdit & e = merged[p.logit_bias_ids[i]];
                    if (e.repeat == 0.f) e = LogitEdit{p.logit_bias_ids[i], 0.f, 1.f, 0.f};
                    e.bias += p.logit_bias_values[i];
                }
                const bool any_penalty = p.repeat_penalty != 1.0f || p.frequency_penalty != 0.0f || p.presence_penalty != 0.0f;
                if (any_penalty && !req.history.empty()) {
                    const size_t window = p.penalty_window == 0 ? req.history.size() : std::min<size_t>(p.penalty_window, req.history.size());
                    std::map<int32_t, int32_t> counts;
                    for (size_t i = req.history.size() - window; i < req.history.size(); ++i) counts[req.history[i]]++;
                    for (const auto & c : counts) {
                        LogitEdit & e = merged[c.first];
                        if (e.repeat == 0.f) e = LogitEdit{c.first, 0.f, 1.f, 0.f};
                        e.repeat = p.repeat_penalty;
                        e.subtract = (float)c.second * p.frequency_penalty + (float)(c.second > 0) * p.presence_penalty;
                    }
                }
                for (const auto & e : merged) edits.push_back(e.second);
                d.edit_end = (uint32_t)edits.size();
                if (p.top_k == 1 && merged.empty() && !p.grammar && forced_token < 0) {
                    d.flags |= 4u;      // plain greedy: arg-max of the raw row, no working copy
                    ++n_greedy_fast;
                } else {
                    any_v2 = true;
                }
            } else {
                d.temperature = row.v1.temperature;
                d.top_p = row.v1.top_p;
                d.top_k = 0;
                d.min_p = 0.f;
                d.flags = 0;
            }
        }
    }

    size_t off_rows = 0;
    size_t off_tokens = align_up(off_rows + R * sizeof(RowDesc), 16);
    size_t off_patches = align_up(off_tokens + T * 4, 16);
    size_t off_copies = align_up(off_patches + patches.size() * 4, 16);
    size_t off_descs = align_up(off_copies + copies.size() * 4, 16);
    size_t off_edits = align_up(off_descs + S * sizeof(SampleDesc), 16);
    size_t off_masks = align_up(off_edits + edits.size() * sizeof(LogitEdit), 16);
    size_t stage_total = align_up(off_masks + masks.size() * sizeof(uint32_t), 16);
    if (stage_total > stage_bytes_) {
        if (h_stage_) cudaFreeHost(h_stage_);
        h_stage_ = nullptr;
        stage_bytes_ = std::max(stage_total * 2, (size_t)1 << 16);
        RB_CUDA(cudaMallocHost(&h_stage_, stage_bytes_));
        d_stage_.ensure(stage_bytes_);
    }
    RowDesc * h_rows = reinterpret_cast<RowDesc *>(h_stage_ + off_rows);
    int32_t * h_tokens = reinterpret_cast<int32_t *>(h_stage_ + off_tokens);
    bool any_adapter = false;
    {
        size_t t = 0;
        for (size_t r = 0; r < R; ++r) {
            const EffRow & row = rows[r];
            RowDesc & d = h_rows[r];
            d.slot = row.slot;
            d.n = (int32_t)row.n;
            d.pos0 = row.pos0;
            d.sample = row.sample ? 1 : 0;
            d.adapter = -1;
            // 0 = the active adapter of the one-at-a-time family (the base model when none is active)
            const int32_t effective = row.adapter > 0 ? row.adapter : row.adapter == 0 ? active_id_ : 0;
            if (effective > 0) {
                d.adapter = adapter_index_.at(effective);
                any_adapter = true;
            }
            d.pos_min = kv->slot(row.slot).pos_min;
            d.pad0 = d.pad1 = 0;
            std::memcpy(h_tokens + t, row.tokens, row.n * 4);
            t += row.n;
        }
    }
#ifdef RETRO_B200_CHECKED
    // Test hook of the bounds-checked build only: RB200_CHECK_INJECT=token puts an id past the vocabulary into
    // the staged plan AFTER validation, =block a block id past the pool into the first queued table patch, so
    // that a test can watch the device-side checks catch them (the accesses are skipped, nothing faults).
    if (const char * inject = std::getenv("RB200_CHECK_INJECT")) {
        if (std::string(inject) == "token") h_tokens[0] = (int32_t)hp.vocab + 7;
        if (std::string(inject) == "block" && patches.size() >= 2) patches[1] = (int32_t)kv->n_blocks() + 3;
    }
#endif
    if (!patches.empty()) std::memcpy(h_stage_ + off_patches, patches.data(), patches.size() * 4);
    if (!copies.empty()) std::memcpy(h_stage_ + off_copies, copies.data(), copies.size() * 4);
    if (S) std::memcpy(h_stage_ + off_descs, descs.data(), S * sizeof(SampleDesc));
    if (!edits.empty()) std::memcpy(h_stage_ + off_edits, edits.data(), edits.size() * sizeof(LogitEdit));
    if (!masks.empty()) std::memcpy(h_stage_ + off_masks, masks.data(), masks.size() * sizeof(uint32_t));
    // (the two lists are cleared once the step's work is enqueued: if anything on the host fails before that,
    // they are still queued and travel with the next step, so the device table cannot fall behind the host's)
    const int n_patches = (int)(patches.size() / 2), n_copies = (int)(copies.size() / 2);

    // result buffer: [SampleOut x S][top ids S x stride][top logprobs S x stride]
    const size_t res_ids = align_up(S * sizeof(SampleOut), 16);
    const size_t res_lps = align_up(res_ids + S * top_stride * 4, 16);
    const size_t res_total = align_up(res_lps + S * top_stride * 4, 16) + 16;
    if (res_total > result_bytes_) {
        if (h_result_) cudaFreeHost(h_result_);
        h_result_ = nullptr;
        result_bytes_ = std::max(res_total * 2, (size_t)1 << 16);
        RB_CUDA(cudaMallocHost(&h_result_, result_bytes_));
        d_result_.ensure(result_bytes_);
    }
    if (S) {
        logits.ensure(S * (size_t)hp.vocab);
        hs_.ensure(S * (size_t)hp.d);
        hs_split_.ensure(S, hp.d);
        if (any_v2) logits_work_.ensure(S * (size_t)hp.vocab);
        if (n_greedy_fast) sample_scratch_.ensure(sample_scratch_bytes((int)hp.vocab, (int)S));
    }
    if (any_adapter) {
        lora_tmp_.ensure((size_t)kLoraTcMaxTargets * kLoraTcMaxSplits * T * (size_t)std::max<uint32_t>(r_max_, 1));
        lora_offsets_.ensure(adapters_.size() + 1);
        lora_sorted_.ensure(T);
    }

    // Attention work items by width in query vectors (tokens x heads of the GQA group): more than 16 go
    // to the tile kernel, 9..16 to the 16-row decode kernel, at most 8 to the eight-column kernel.
    int n_attn_items = 0, n_small_items = 0, max_ctx = 1;
    bool any_wide_item = false, any_mid_item = false;
    const int attn_group = (int)(hp.n_head / hp.n_head_kv);
    const bool use_decode8 = attn_decode8_ && attention_decode8_supported((int)hp.n_head, (int)hp.n_head_kv, (int)hp.head_dim, (int)kBlockTokens);
    for (size_t r = 0; r < R; ++r) {
        const int n = (int)rows[r].n, tail = n % attn_tile_tokens_;
        n_attn_items += (n + attn_tile_tokens_ - 1) / attn_tile_tokens_;
        if (n >= attn_tile_tokens_ && attn_tile_tokens_ * attn_group > 16) any_wide_item = true;
        if (n >= attn_tile_tokens_ && attn_tile_tokens_ * attn_group <= 16) any_mid_item = true;
        if (tail) {
            const int cols = tail * attn_group;
            if (cols > 16) any_wide_item = true;
            else if (cols > 8 || !use_decode8) any_mid_item = true;
            else ++n_small_items;
        }
        max_ctx = std::max(max_ctx, (int)rows[r].pos0 + n);
    }
    // few small items: cut each sequence's KV blocks over several CTAs so the GPU is still full
    int attn_splits = 1;
    if (n_small_items > 0) {
        // two CTAs of the split-KV kernel fit an SM (shared memory): as many splits as keep the grid within one
        // wave - rounding up left a second, nearly empty wave (16 requests: 384 CTAs on 296 places, 6.0 -> 5.7 ms per step)
        const int want = (2 * n_sm_) / (n_small_items * (int)hp.n_head_kv);
        attn_splits = std::max(1, std::min({want, attention_decode8_max_splits(), (max_ctx / (int)kBlockTokens) / 8}));
        if (attn_splits > 1)
            attn_scratch_.ensure(attention_decode8_scratch_floats(n_attn_items, (int)hp.n_head_kv, attn_splits, (int)hp.head_dim));
    }

    // Quantised pools: decode rows are read from the pool by attention_decode8's own Q8_0 / Q4_0 kernel; every other row
    // needs its context in the f16 scratch.
    const int pool_read_tokens = kv_storage_ != KV_F16 && use_decode8 && kv_q8_native_ ? 8 / attn_group : 0;
    const bool kv_scratch_needed = kv_storage_ != KV_F16 && (any_wide_item || any_mid_item || pool_read_tokens == 0);
    int n_scratch_rows = 0;
    if (kv_scratch_needed)
        for (size_t r = 0; r < R; ++r) n_scratch_rows += (int)rows[r].n > pool_read_tokens ? 1 : 0;

    // ---- device work. Everything the launches depend on besides the contents of the staging buffer
    // is in `sig`: a step whose signature was seen before is replayed as a CUDA graph (one launch
    // instead of hundreds), captured the second time the signature occurs - the first time runs
    // eagerly, so every lazy allocation and kernel attribute is in place before a capture.
    last_h2d_bytes = stage_total;
    last_d2h_bytes = S ? res_total - 16 : 0;
    const std::vector<uint64_t> sig = {R, T, S, (uint64_t)n_patches, (uint64_t)n_copies, edits.size(), top_stride, any_v2, (uint64_t)n_greedy_fast,
                                       any_adapter, (uint64_t)n_attn_items, (uint64_t)n_small_items, any_wide_item, any_mid_item,
                                       (uint64_t)attn_splits, stage_total, res_total, (uint64_t)result_bytes_, (uint64_t)adapters_.size(), (uint64_t)masks.size(),
                                       // a quantised pool's dequantisation grid covers the longest row's blocks
                                       kv_scratch_needed ? (uint64_t)((max_ctx + kBlockTokens - 1) / kBlockTokens) : 0, (uint64_t)n_scratch_rows};
    auto issue = [&]() {
    last_launches = 0;
    RB_CUDA(cudaMemcpyAsync(d_stage_.ptr, h_stage_, stage_total, cudaMemcpyHostToDevice, stream));
    const RowDesc * d_rows = reinterpret_cast<const RowDesc *>(d_stage_.ptr + off_rows);
    const int32_t * d_tokens = reinterpret_cast<const int32_t *>(d_stage_.ptr + off_tokens);
    const KvLayout kvl = kv_layout();
    // what the decode-row kernel sees: the quantised pool itself, or (storage F16) the pool / its dequantised scratch
    KvLayout kv_rows = kvl;
    if (!kv_q8_native_) kv_rows.storage = KV_F16;
#define RB_K(cls, n, ...)            \
    do {                             \
        prof_.begin(cls, stream);    \
        __VA_ARGS__;                 \
        prof_.end(cls, n, stream);   \
        last_launches += (n);        \
    } while (0)
    if (n_patches) {
        RB_K(K_OTHER, 1, launch_block_table_patch(block_table_.ptr, reinterpret_cast<const int32_t *>(d_stage_.ptr + off_patches), n_patches, stream,
                                                  (int)block_table_.count, (int)kv->n_blocks(), check_word_.ptr));
    }
    if (n_copies) {
        RB_K(K_OTHER, 1, launch_kv_block_copy(kvl, (int)hp.n_layer, reinterpret_cast<const int32_t *>(d_stage_.ptr + off_copies), n_copies, stream));
    }
    maps.n_adapters = (int32_t)adapters_.size();
    RB_K(K_PACK, 2, launch_pack(d_rows, (int)R, (int)T, block_table_.ptr, kvl.max_blocks, kvl.block_tokens, attn_tile_tokens_, maps, stream));
    cur_tok_adapter_ = maps.tok_adapter;
    cur_any_adapter_ = any_adapter;
    if (any_adapter && adapters_.size() <= 1024) {
        // the step's tokens grouped by adapter, once for every target and layer
        RB_K(K_LORA, 1, launch_moe_group(maps.tok_adapter, (int)T, (int)adapters_.size(), lora_offsets_.ptr, lora_sorted_.ptr, stream));
    }

    const int d = (int)hp.d, dq = (int)hp.dq(), dkv = (int)hp.dkv(), ldqkv = dq + 2 * dkv, ff = (int)hp.ff;
    const int Ti = (int)T;
    RB_K(K_OTHER, 1, launch_embed(model->token_embd, d_tokens, Ti, x_.ptr, stream, check_word_.ptr));
    bool norm_done = false;         // this layer's attention norm was already written by the previous layer's down projection
    for (uint32_t l = 0; l < hp.n_layer; ++l) {
        const LayerWeights & lw = model->layers[l];
        const std::string p = "blk." + std::to_string(l) + ".";
        // the f32 copy of an activation is written only when something other than a split-reading GEMM consumes it
        const bool qkv_split = !any_adapter && lw.wqkv.data && linear_reads_split(lw.wqkv, d, Ti, xn_split_.get());
        if (!norm_done)
            RB_K(K_OTHER, 1, launch_rms_norm(x_.ptr, d, nullptr, lw.attn_norm, d, hp.eps, qkv_split ? nullptr : xn_.ptr, d, Ti, stream, xn_split_.get()));
        norm_done = false;
        const RopeStoreArgs rope_args{(int)hp.n_head, (int)hp.n_head_kv, (int)hp.head_dim, (int)hp.n_rot, hp.neox, model->inv_freq.ptr,
                                      maps.tok_pos,   maps.tok_cell,     kvl,              (int)l};
        bool roped = false;
        if (lw.wqkv.data) {
            // RoPE and the KV store by the projection's finish kernel when nothing else touches q, k, v in between
            FinishTail rope_tail;
            rope_tail.kind = 3;
            rope_tail.rope = &rope_args;
            roped = linear(lw.wqkv, xn_.ptr, d, Ti, qkv_.ptr, ldqkv, lw.bqkv, nullptr, 0, xn_split_.get(), any_adapter || lw.q_norm ? nullptr : &rope_tail);
        } else {
            linear(lw.wq, xn_.ptr, d, Ti, qkv_.ptr, ldqkv, lw.bqkv, nullptr, 0);
            linear(lw.wk, xn_.ptr, d, Ti, qkv_.ptr + dq, ldqkv, lw.bqkv ? lw.bqkv + dq : nullptr, nullptr, 0);
            linear(lw.wv, xn_.ptr, d, Ti, qkv_.ptr + dq + dkv, ldqkv, lw.bqkv ? lw.bqkv + dq + dkv : nullptr, nullptr, 0);
        }
        if (any_adapter) {
            lora_group({p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"}, {0, dq, dq + dkv}, xn_.ptr, d, Ti, qkv_.ptr, ldqkv);
        }
        if (lw.q_norm) {
            RB_K(K_OTHER, 2, launch_rms_norm(qkv_.ptr, ldqkv, nullptr, lw.q_norm, dq, hp.eps, qkv_.ptr, ldqkv, Ti, stream);
                 launch_rms_norm(qkv_.ptr + dq, ldqkv, nullptr, lw.k_norm, dkv, hp.eps, qkv_.ptr + dq, ldqkv, Ti, stream));
        }
        if (!roped) RB_K(K_OTHER, 1, launch_rope_store(qkv_.ptr, ldqkv, Ti, rope_args, stream));
        if (kv_storage_ != KV_F16) {
            // the rotated K and the V rows are still in the qkv buffer: quantise them into the pool, then bring every
            // block the step's rows attend to (the new cells included, now as the pool holds them) into the f16 scratch
            RB_K(K_ATTN, kv_scratch_needed ? 2 : 1, launch_kv_quant_store(qkv_.ptr, ldqkv, Ti, (int)hp.n_head, kvl, (int)l, maps.tok_cell, stream);
                 if (kv_scratch_needed)
                     launch_kv_dequant(kvl, (int)l, (int)R, n_scratch_rows, (max_ctx + (int)kBlockTokens - 1) / (int)kBlockTokens, maps.cu_rows, maps.tok_slot,
                                       maps.tok_pos, maps.tok_pos_min, pool_read_tokens, stream));
        }
        if (attn_mma_) {
            // every row of the step goes through the split-KV kernel: its merge writes the split form as well
            const bool merge_splits = fused_finish_ && att_split_.get() && !any_wide_item && !any_mid_item && n_small_items && attn_splits > 1 &&
                                      hp.head_dim % 32 == 0;
            // Decode rows (HBM-bound, many small CTAs) and prefill tiles (tensor-bound, one CTA per SM and a ragged
            // last wave) touch disjoint rows: with both in a step the decode kernel runs on a second stream
            // beside the tile kernel and fills the SMs its tail leaves idle.
            const bool overlap = attn_overlap_ && any_wide_item && n_small_items > 0;
            cudaStream_t small_stream = overlap ? side_stream_ : stream;
            RB_K(K_ATTN, (any_wide_item ? 1 : 0) + (any_mid_item ? 1 : 0) + (n_small_items ? (attn_splits > 1 ? 2 : 1) : 0),
                 if (overlap) {
                     RB_CUDA(cudaEventRecord(ev_fork_, stream));
                     RB_CUDA(cudaStreamWaitEvent(side_stream_, ev_fork_, 0));
                     launch_attention_decode8(qkv_.ptr, ldqkv, (int)hp.n_head, kv_rows, (int)l, maps.attn_items, n_attn_items, maps.tok_slot, maps.tok_pos,
                                              maps.tok_pos_min, att_.ptr, dq, attn_splits, attn_scratch_.ptr, small_stream, nullptr);
                     RB_CUDA(cudaEventRecord(ev_join_, side_stream_));
                 }
                 if (any_wide_item && attn_tc5_)
                     launch_attention_tc5(qkv_.ptr, ldqkv, (int)hp.n_head, kvl, (int)l, attn_maps_, maps.attn_items, n_attn_items, maps.tok_slot,
                                          maps.tok_pos, maps.tok_pos_min, att_.ptr, dq, true, device_error_.ptr, stream);
                 else if (any_wide_item)
                     launch_attention_mma(qkv_.ptr, ldqkv, (int)hp.n_head, kvl, (int)l, maps.attn_items, n_attn_items, maps.tok_slot, maps.tok_pos,
                                          maps.tok_pos_min, att_.ptr, dq, true, stream);
                 if (any_mid_item) launch_attention_decode(qkv_.ptr, ldqkv, (int)hp.n_head, kvl, (int)l, maps.attn_items, n_attn_items, maps.tok_slot,
                                                           maps.tok_pos, maps.tok_pos_min, att_.ptr, dq, use_decode8 ? 8 : 0, stream);
                 if (n_small_items && !overlap) launch_attention_decode8(qkv_.ptr, ldqkv, (int)hp.n_head, kv_rows, (int)l, maps.attn_items, n_attn_items,
                                                                         maps.tok_slot, maps.tok_pos, maps.tok_pos_min, att_.ptr, dq, attn_splits,
                                                                         attn_scratch_.ptr, stream, merge_splits ? att_split_.get() : nullptr);
                 if (overlap) RB_CUDA(cudaStreamWaitEvent(stream, ev_join_, 0)));
            if (att_split_.get() && !merge_splits) RB_K(K_OTHER, 1, launch_split_prep(att_.ptr, dq, dq, Ti, att_split_.view, stream));
        } else {
            RB_K(K_ATTN, 1, launch_attention_ref(qkv_.ptr, ldqkv, Ti, (int)hp.n_head, kvl, (int)l, maps.tok_slot, maps.tok_pos, maps.tok_pos_min,
                                                 att_.ptr, dq, stream, att_split_.get()));
            // the reference kernel writes the split form itself only when a head is whole 32-column sub-blocks
            if (att_split_.get() && hp.head_dim % 32 != 0) RB_K(K_OTHER, 1, launch_split_prep(att_.ptr, dq, dq, Ti, att_split_.view, stream));
        }
        // x = x + Wo att, then the FFN's norm of x: by the projection's finish kernel where it has one
        const bool gu_split = !any_adapter && hp.n_expert == 0 && lw.wgu.data && linear_reads_split(lw.wgu, d, Ti, xn_split_.get());
        FinishTail ffn_norm_tail;
        ffn_norm_tail.kind = 1;
        ffn_norm_tail.norm_w = lw.ffn_norm;
        ffn_norm_tail.eps = hp.eps;
        ffn_norm_tail.out = gu_split ? nullptr : xn_.ptr;
        ffn_norm_tail.ld_out = d;
        if (xn_split_.get()) ffn_norm_tail.split = *xn_split_.get();
        const bool ffn_normed = linear(lw.wo, att_.ptr, dq, Ti, x_.ptr, d, nullptr, x_.ptr, d, att_split_.get(), any_adapter ? nullptr : &ffn_norm_tail);
        if (any_adapter) lora(p + "attn_output.weight", att_.ptr, dq, Ti, x_.ptr, d);
        if (!ffn_normed)
            RB_K(K_OTHER, 1, launch_rms_norm(x_.ptr, d, nullptr, lw.ffn_norm, d, hp.eps, gu_split ? nullptr : xn_.ptr, d, Ti, stream, xn_split_.get()));
        if (hp.n_expert == 0) {
            const bool down_split = !any_adapter && linear_reads_split(lw.wdown, ff, Ti, hff_split_.get());
            bool activated = false;
            if (lw.wgu.data) {
                FinishTail act_tail;
                act_tail.kind = 2;
                act_tail.out = down_split ? nullptr : hff_.ptr;
                act_tail.ld_out = ff;
                if (hff_split_.get()) act_tail.split = *hff_split_.get();
                activated = linear(lw.wgu, xn_.ptr, d, Ti, gu_.ptr, 2 * ff, nullptr, nullptr, 0, xn_split_.get(), any_adapter ? nullptr : &act_tail);
            } else {
                linear(lw.wgate, xn_.ptr, d, Ti, gu_.ptr, 2 * ff, nullptr, nullptr, 0);
                linear(lw.wup, xn_.ptr, d, Ti, gu_.ptr + ff, 2 * ff, nullptr, nullptr, 0);
            }
            if (any_adapter) {
                lora_group({p + "ffn_gate.weight", p + "ffn_up.weight"}, {0, ff}, xn_.ptr, d, Ti, gu_.ptr, 2 * ff);
            }
            if (!activated) RB_K(K_OTHER, 1, launch_swiglu(gu_.ptr, 2 * ff, ff, Ti, down_split ? nullptr : hff_.ptr, ff, stream, hff_split_.get()));
            // x = x + Wdown h, then the next layer's attention norm of x
            FinishTail next_norm_tail;
            const bool has_next = l + 1 < hp.n_layer && !any_adapter;
            if (has_next) {
                const LayerWeights & nw = model->layers[l + 1];
                const bool next_qkv_split = nw.wqkv.data && linear_reads_split(nw.wqkv, d, Ti, xn_split_.get());
                next_norm_tail.kind = 1;
                next_norm_tail.norm_w = nw.attn_norm;
                next_norm_tail.eps = hp.eps;
                next_norm_tail.out = next_qkv_split ? nullptr : xn_.ptr;
                next_norm_tail.ld_out = d;
                if (xn_split_.get()) next_norm_tail.split = *xn_split_.get();
            }
            norm_done = linear(lw.wdown, hff_.ptr, ff, Ti, x_.ptr, d, nullptr, x_.ptr, d, hff_split_.get(), has_next ? &next_norm_tail : nullptr);
            if (any_adapter) lora(p + "ffn_down.weight", hff_.ptr, ff, Ti, x_.ptr, d);
        } else {
            const int E = (int)hp.n_expert, K = (int)hp.n_expert_used, P = Ti * K;
            linear(lw.router, xn_.ptr, d, Ti, router_logits_.ptr, E, nullptr, nullptr, 0);
            RB_K(K_MOE, 1, launch_moe_route(router_logits_.ptr, E, K, Ti, moe_ids_.ptr, moe_w_.ptr, stream));
            RB_CUDA(cudaMemcpyAsync(route_ids.ptr + (size_t)l * P, moe_ids_.ptr, (size_t)P * 4, cudaMemcpyDeviceToDevice, stream));
            if (ep_comm_) {
                // expert parallelism: the pairs travel to their experts' ranks and back
                RB_K(K_MOE, 1, launch_moe_group(moe_ids_.ptr, P, E, moe_offsets_.ptr, moe_sorted_.ptr, stream));
                prof_.begin(K_MOE, stream);
                ep_moe_layer(lw, Ti);
                prof_.end(K_MOE, 8, stream);
                continue;
            }
            if (moe_experts_on_tensor_cores(lw)) {
                // the pairs grouped by expert, then one grouped tensor-core GEMM per projection
                RB_K(K_MOE, 1, launch_moe_group(moe_ids_.ptr, P, E, moe_offsets_.ptr, moe_sorted_.ptr, stream));
                prof_.begin(K_MOE, stream);
                moe_experts_tc(lw, xn_.ptr, d, moe_sorted_.ptr, K, moe_offsets_.ptr, P, pair_y_.ptr, d);
                launch_moe_combine(pair_y_.ptr, d, moe_ids_.ptr, moe_w_.ptr, K, d, Ti, x_.ptr, x_.ptr, stream);
                prof_.end(K_MOE, 8, stream);
                ++last_launches;
                continue;
            }
            // pairs grouped by expert: every expert's weights are streamed once per eight of its pairs
            RB_K(K_MOE, 3, launch_moe_group(moe_ids_.ptr, P, E, moe_offsets_.ptr, moe_sorted_.ptr, stream);
                 launch_moe_gemm_grouped(lw.gate_exps, lw.gate_stride, E, moe_offsets_.ptr, moe_sorted_.ptr, xn_.ptr, d, K, pair_gu_.ptr, 2 * ff, stream);
                 launch_moe_gemm_grouped(lw.up_exps, lw.up_stride, E, moe_offsets_.ptr, moe_sorted_.ptr, xn_.ptr, d, K, pair_gu_.ptr + ff, 2 * ff, stream));
            RB_K(K_OTHER, 1, launch_swiglu(pair_gu_.ptr, 2 * ff, ff, P, pair_h_.ptr, ff, stream));
            RB_K(K_MOE, 2, launch_moe_gemm_grouped(lw.down_exps, lw.down_stride, E, moe_offsets_.ptr, moe_sorted_.ptr, pair_h_.ptr, ff, 1, pair_y_.ptr, d, stream);
                 launch_moe_combine(pair_y_.ptr, d, moe_ids_.ptr, moe_w_.ptr, K, d, Ti, x_.ptr, x_.ptr, stream));
        }
    }
    SampleOut * d_out = reinterpret_cast<SampleOut *>(d_result_.ptr);
    int32_t * d_top_ids = reinterpret_cast<int32_t *>(d_result_.ptr + res_ids);
    float * d_top_lps = reinterpret_cast<float *>(d_result_.ptr + res_lps);
    if (S) {
        RB_K(K_OTHER, 1, launch_rms_norm(x_.ptr, d, maps.out_index, model->output_norm, d, hp.eps, hs_.ptr, d, (int)S, stream, hs_split_.get()));
        linear(model->output, hs_.ptr, d, (int)S, logits.ptr, (int)hp.vocab, model->output_bias, nullptr, 0, hs_split_.get());
        if (any_v2) {
            RB_CUDA(cudaMemcpyAsync(logits_work_.ptr, logits.ptr, S * (size_t)hp.vocab * 4, cudaMemcpyDeviceToDevice, stream));
        }
        RB_K(K_SAMPLE, (n_greedy_fast < (int)S ? 1 : 0) + (n_greedy_fast ? 2 : 0), launch_sample(logits.ptr, any_v2 ? logits_work_.ptr : nullptr, (int)hp.vocab, (int)S,
                                        reinterpret_cast<const SampleDesc *>(d_stage_.ptr + off_descs),
                                        reinterpret_cast<const LogitEdit *>(d_stage_.ptr + off_edits),
                                        masks.empty() ? nullptr : reinterpret_cast<const uint32_t *>(d_stage_.ptr + off_masks), d_out, d_top_ids, d_top_lps,
                                        (int)std::max<size_t>(top_stride, 1), n_greedy_fast, sample_scratch_.ptr, stream));
    }
#undef RB_K
    if (S) RB_CUDA(cudaMemcpyAsync(h_result_, d_result_.ptr, res_total - 16, cudaMemcpyDeviceToHost, stream));
    RB_CUDA(cudaMemcpyAsync(h_result_ + result_bytes_ - 16, device_error_.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream));
    };
#ifdef RETRO_B200_CHECKED
    graphs_enabled_ = false;        // the check word is read back after every step, outside any captured graph
#endif
    run_step_work(sig, issue);
    patches.clear();
    copies.clear();
    const cudaError_t sync = cudaStreamSynchronize(stream);
    if (sync != cudaSuccess) {
        set_error(std::string("the decode failed on the device (") + cudaGetErrorString(sync) +
                  "): the KV may hold a prefix of the submitted tokens (query it with the seq_pos entry point) - do not resubmit tokens "
                  "that are already resident");
        return STATUS_RUNTIME;
    }
    const cudaError_t launch_status = cudaGetLastError();
    if (launch_status != cudaSuccess) {
        set_error(std::string("a kernel of the step failed to launch: ") + cudaGetErrorString(launch_status));
        return STATUS_RUNTIME;
    }
    if (*reinterpret_cast<const int *>(h_result_ + result_bytes_ - 16) != 0) {
        cudaMemsetAsync(device_error_.ptr, 0, sizeof(int), stream);
        set_error("the decode failed on the device: a pipeline wait inside a tensor-core kernel timed out; the KV may hold a prefix of "
                  "the submitted tokens (query it with the seq_pos entry point)");
        return STATUS_RUNTIME;
    }
#ifdef RETRO_B200_CHECKED
    RB_CUDA(cudaMemcpy(last_check, check_word_.ptr, sizeof last_check, cudaMemcpyDeviceToHost));
    if (last_check[0] != 0) {
        static const char * const what[] = {"", "a token id", "a slot", "a position", "a block-table index", "a physical block id", "a KV cell", "an adapter index"};
        const int code = last_check[0] >= 1 && last_check[0] <= 7 ? last_check[0] : 0;
        RB_CUDA(cudaMemset(check_word_.ptr, 0, 4 * sizeof(int)));
        set_error(std::string("bounds-checked build: ") + what[code] + " read on the device was " + std::to_string(last_check[1]) + ", outside [0, " +
                  std::to_string(last_check[2]) + ") (" + std::to_string(last_check[3]) + " violations in this step); the accesses were skipped, the KV may hold a "
                  "prefix of the submitted tokens");
        return STATUS_RUNTIME;
    }
#endif
    cudaEventElapsedTime(&last_ms, ev_begin_, ev_end_);
    prof_.collect();
    last_T = T;
    last_S = S;
    last_R = R;

    if (hp.n_expert && route_enabled) {
        const size_t P = T * hp.n_expert_used;
        std::vector<int32_t> ids((size_t)hp.n_layer * P);
        RB_CUDA(cudaMemcpy(ids.data(), route_ids.ptr, ids.size() * 4, cudaMemcpyDeviceToHost));
        for (uint32_t l = 0; l < hp.n_layer; ++l)
            for (size_t i = 0; i < P; ++i) ++route_counts[l][ids[(size_t)l * P + i]];
        route_pairs += ids.size();      // every pair is served from a bank resident on the device
    }

    if (forced_outside_grammar) {
        set_error("the reasoning budget forced a token excluded by the grammar");
        return STATUS_RUNTIME;
    }
    if (grammar_dead_end) {
        // as in the reference, the decode has happened by the time a grammar turns out to allow nothing (retro_gen_core.cpp:790-797)
        set_error("grammar allows no token at this position");
        return STATUS_RUNTIME;
    }

    // ---- outputs
    const SampleOut * h_out = reinterpret_cast<const SampleOut *>(h_result_);
    const int32_t * h_ids = reinterpret_cast<const int32_t *>(h_result_ + res_ids);
    const float * h_lps = reinterpret_cast<const float *>(h_result_ + res_lps);
    size_t s = 0;
    for (size_t r = 0; r < R; ++r) {
        const EffRow & row = rows[r];
        OutRow & o = out_rows[r];
        o = OutRow{};
        if (!row.sample) continue;
        const SampleOut & so = h_out[s];
        RequestState & req = requests[row.request];
        // a forcing budget machine had its token reported by the sampling kernel; here it moves on
        bool forced = false;
        const int32_t emitted = req.budget.next(so.token, forced);
        o.token = emitted;
        o.logprob = so.logprob;
        o.sampled = 1;
        o.forced = forced ? 1 : 0;
        o.n_top = so.n_top;
        o.sampled_logprob = row.v2 && row.want_logprob ? so.sampled_logprob : 0.f;
        for (uint32_t j = 0; j < so.n_top; ++j) {
            out_top_ids[r * n_top_stride + j] = h_ids[s * top_stride + j];
            out_top_logprobs[r * n_top_stride + j] = h_lps[s * top_stride + j];
        }
        ++req.draws;
        if (row.v2) req.history.push_back(emitted);
        // the request's grammar follows the emitted token; a row without one drops what the request had
        if (row_grammar[r]) {
            row_grammar[r]->advance(model->piece(emitted, false), model->is_eog(emitted));
            req.grammar = std::move(row_grammar[r]);
        } else if (row.v2) {
            req.grammar.reset();
        }
        ++s;
    }
    return STATUS_OK;
}

// ---------------------------------------------------------------------------------------------
// Reasoning budget (reference: retro_engine_set_reasoning_budget, retro_chat_parser.cpp:544-640)

int Engine::set_reasoning_tags(const int32_t * start, size_t n_start, const int32_t * const * ends, const size_t * n_ends, size_t n_end_tags,
                               size_t n_prompt_tail) {
    ReasoningPlan plan;
    auto tag = [&](const int32_t * tokens, size_t n, std::vector<int32_t> & out) {
        for (size_t i = 0; i < n; ++i) {
            if (tokens[i] < 0 || (uint32_t)tokens[i] >= model->hp.vocab) return false;
            out.push_back(tokens[i]);
        }
        return true;
    };
    std::vector<int32_t> one;
    if (n_start && (!start || !tag(start, n_start, one))) {
        set_error("a reasoning tag holds a token id outside the vocabulary");
        return STATUS_RUNTIME;
    }
    if (!one.empty()) plan.starts.push_back(one);
    for (size_t e = 0; e < n_end_tags; ++e) {
        one.clear();
        if (n_ends[e] && (!ends || !ends[e] || !tag(ends[e], n_ends[e], one))) {
            set_error("a reasoning tag holds a token id outside the vocabulary");
            return STATUS_RUNTIME;
        }
        if (!one.empty()) plan.ends.push_back(one);
    }
    plan.n_prompt_tail = n_prompt_tail;
    plan.budget = reasoning_plan_.budget;
    if (!plan.ends.empty()) plan.forced = plan.ends.front();
    plan.active = plan.budget >= 0 && !plan.starts.empty() && !plan.ends.empty();
    reasoning_plan_ = std::move(plan);
    return STATUS_OK;
}

int Engine::set_reasoning_budget(int32_t budget) {
    if (budget < -1) {
        set_error("reasoning budget must be -1 (the model decides) or a token count");
        return STATUS_RUNTIME;
    }
    if (budget >= 0 && (reasoning_plan_.starts.empty() || reasoning_plan_.ends.empty())) {
        // the reference derives the tags from the model's chat template; here the caller's template layer hands
        // them over first (retro_b200_engine_set_reasoning_tags), and without them there is nothing to limit
        set_error("the chat template declares no reasoning block, so a reasoning budget has nothing to limit");
        return STATUS_RUNTIME;
    }
    reasoning_plan_.budget = budget;
    reasoning_plan_.active = budget >= 0;
    return STATUS_OK;
}

// ---------------------------------------------------------------------------------------------
// Sequence memory

int Engine::seq_rm(int32_t slot, int32_t p0, int32_t p1) {
    if (slot < 0 || slot >= (int32_t)config.n_seq_max) {
        set_error("slot is outside the context's sequence range");
        return STATUS_RUNTIME;
    }
    if (!kv->seq_rm(slot, p0, p1)) {
        set_error("the memory cannot remove that partial range; remove the whole sequence instead");
        return STATUS_RUNTIME;
    }
    return STATUS_OK;
}

int Engine::seq_cp(int32_t src, int32_t dst, int32_t p0, int32_t p1) {
    const int32_t n = (int32_t)config.n_seq_max;
    if (src < 0 || src >= n || dst < 0 || dst >= n) {
        set_error("seq_cp slots are outside the context's sequence range");
        return STATUS_RUNTIME;
    }
    if (!config.kv_unified && !(p0 <= 0 && p1 < 0)) {
        set_error("a partitioned KV pool only supports whole-sequence copies");
        return STATUS_RUNTIME;
    }
    if (kv->seq_cp(src, dst, p0, p1) == KvManager::DST_NOT_EMPTY) {
        set_error("the destination slot of a seq_cp must be empty: remove it first with seq_rm");
        return STATUS_RUNTIME;
    }
    flush_kv_updates();
    return STATUS_OK;
}

int Engine::seq_pos(int32_t slot, int32_t * pmin, int32_t * pmax) {
    if (!pmin || !pmax) {
        set_error("the position outputs are required");
        return STATUS_RUNTIME;
    }
    if (slot < 0 || slot >= (int32_t)config.n_seq_max) {
        set_error("slot is outside the context's sequence range");
        return STATUS_RUNTIME;
    }
    const KvSlot & s = kv->slot(slot);
    *pmin = s.empty() ? -1 : s.pos_min;
    *pmax = s.empty() ? -1 : s.pos_max;
    return STATUS_OK;
}

namespace {
struct SnapshotHeader {
    char magic[8];
    uint32_t version;
    uint32_t n_layer, n_head_kv, head_dim;
    int32_t pos_min, pos_max;
    uint64_t payload_bytes;
    uint64_t checksum;
};
const char kSnapshotMagic[8] = {'R', 'B', '2', 'K', 'V', 'S', 'N', 'P'};
} // namespace

int Engine::seq_save(int32_t slot, uint32_t flags, uint8_t * buffer, size_t n_buffer, size_t * out_n) {
    if (!out_n) {
        set_error("out_n_bytes is required");
        return STATUS_RUNTIME;
    }
    if (flags & ~RETRO_STATE_SEQ_FLAGS_PARTIAL_ONLY) {
        set_error("only host snapshots (flags 0 or PARTIAL_ONLY) are supported");
        return STATUS_RUNTIME;
    }
    if (slot < 0 || slot >= (int32_t)config.n_seq_max) {
        set_error("slot is outside the context's sequence range");
        return STATUS_RUNTIME;
    }
    const HParams & hp = model->hp;
    const KvSlot & s = kv->slot(slot);
    // A dense attention model has no partial (recurrent) state: a PARTIAL_ONLY snapshot is a bare header.
    const bool partial = (flags & RETRO_STATE_SEQ_FLAGS_PARTIAL_ONLY) != 0;
    const size_t n_pos = (s.empty() || partial) ? 0 : (size_t)(s.pos_max - s.pos_min + 1);
    // per position, layer and K | V: the heads' rows as the pool holds them (f16 values, or quantised rows)
    const size_t pos_bytes = (size_t)hp.n_layer * 2 * hp.n_head_kv * kv_row_bytes(kv_storage_, (int)hp.head_dim);
    const size_t payload = n_pos * pos_bytes;
    const size_t required = sizeof(SnapshotHeader) + payload;
    *out_n = required;
    if (!buffer) return STATUS_OK;
    if (n_buffer < required) {
        set_error("the save buffer is too small for this sequence's state");
        return STATUS_BUFFER_TOO_SMALL;
    }
    SnapshotHeader h{};
    std::memcpy(h.magic, kSnapshotMagic, 8);
    h.version = (partial ? 2 : 1) + 16 * (uint32_t)kv_storage_;       // a snapshot only loads into a pool of its storage type
    h.n_layer = hp.n_layer;
    h.n_head_kv = hp.n_head_kv;
    h.head_dim = hp.head_dim;
    h.pos_min = n_pos ? s.pos_min : -1;
    h.pos_max = n_pos ? s.pos_max : -1;
    h.payload_bytes = payload;
    if (n_pos) {
        DeviceBuffer<__half> dense;
        dense.in_graphs = false;
        dense.ensure(payload / sizeof(__half));
        launch_kv_snapshot(kv_layout(), (int)hp.n_layer, block_table_.ptr + (size_t)slot * kv->max_blocks(), s.pos_min, (int)n_pos, dense.ptr, false,
                           stream);
        RB_CUDA(cudaMemcpyAsync(buffer + sizeof h, dense.ptr, payload, cudaMemcpyDeviceToHost, stream));
        RB_CUDA(cudaStreamSynchronize(stream));
    }
    h.checksum = fnv1a(buffer + sizeof h, payload);
    std::memcpy(buffer, &h, sizeof h);
    return STATUS_OK;
}

int Engine::seq_load(int32_t slot, uint32_t flags, const uint8_t * buffer, size_t n_bytes, size_t * out_read) {
    if (!out_read) {
        set_error("out_n_read is required");
        return STATUS_RUNTIME;
    }
    if (flags & ~RETRO_STATE_SEQ_FLAGS_PARTIAL_ONLY) {
        set_error("only host snapshots (flags 0 or PARTIAL_ONLY) are supported");
        return STATUS_RUNTIME;
    }
    if (slot < 0 || slot >= (int32_t)config.n_seq_max) {
        set_error("slot is outside the context's sequence range");
        return STATUS_RUNTIME;
    }
    if (!buffer || n_bytes == 0) {
        set_error("a snapshot buffer is required");
        return STATUS_RUNTIME;
    }
    const HParams & hp = model->hp;
    const char * refused = "the snapshot was refused (wrong size, flags or corrupted data)";
    SnapshotHeader h{};
    if (n_bytes < sizeof h) { set_error(refused); return STATUS_RUNTIME; }
    std::memcpy(&h, buffer, sizeof h);
    const bool partial = (flags & RETRO_STATE_SEQ_FLAGS_PARTIAL_ONLY) != 0;
    if (std::memcmp(h.magic, kSnapshotMagic, 8) != 0 || h.version != (partial ? 2u : 1u) + 16u * (uint32_t)kv_storage_ || h.n_layer != hp.n_layer ||
        h.n_head_kv != hp.n_head_kv || h.head_dim != hp.head_dim || n_bytes < sizeof h + h.payload_bytes) {
        set_error(refused);
        return STATUS_RUNTIME;
    }
    const size_t n_pos = h.pos_min < 0 ? 0 : (size_t)(h.pos_max - h.pos_min + 1);
    if (h.payload_bytes != n_pos * hp.n_layer * 2 * hp.n_head_kv * kv_row_bytes(kv_storage_, (int)hp.head_dim) || fnv1a(buffer + sizeof h, h.payload_bytes) != h.checksum ||
        (n_pos && (h.pos_min < 0 || (uint32_t)h.pos_max >= n_ctx_seq))) {
        set_error(refused);
        return STATUS_RUNTIME;
    }
    if (n_pos) {
        if (!kv->slot(slot).empty()) kv->seq_rm(slot, -1, -1);
        kv->begin();
        if (kv->reserve(slot, h.pos_min, (int32_t)n_pos) != KvManager::OK) {
            kv->rollback();
            set_error("the KV cache is full: no free block for the snapshot");
            return STATUS_RUNTIME;
        }
        kv->commit();
        flush_kv_updates();
        DeviceBuffer<__half> dense;
        dense.in_graphs = false;
        dense.ensure(h.payload_bytes / sizeof(__half));
        RB_CUDA(cudaMemcpyAsync(dense.ptr, buffer + sizeof h, h.payload_bytes, cudaMemcpyHostToDevice, stream));
        launch_kv_snapshot(kv_layout(), (int)hp.n_layer, block_table_.ptr + (size_t)slot * kv->max_blocks(), h.pos_min, (int)n_pos, dense.ptr, true,
                           stream);
        RB_CUDA(cudaStreamSynchronize(stream));
    }
    *out_read = sizeof h + h.payload_bytes;
    return STATUS_OK;
}

int Engine::memory(retro_engine_memory_info * out) {
    if (!out) {
        set_error("out is required");
        return STATUS_RUNTIME;
    }
    out->struct_size = sizeof(retro_engine_memory_info);
    out->n_slots = config.n_seq_max;
    out->cells_total = config.n_ctx;
    out->cells_used = kv->cells_used();
    out->kv_bytes = (kcache_.count + vcache_.count) * sizeof(__half) + kq_.count + vq_.count;
    out->recurrent_bytes = 0;
    return STATUS_OK;
}

// ---------------------------------------------------------------------------------------------
// Per-row adapters

// Reads a LoRA adapter GGUF (general.type = adapter, adapter.type = lora, tensors <weight>.lora_a [in, r]
// and <weight>.lora_b [r, out]) into F32 host copies; false with the error set when it is refused.
bool Engine::read_adapter_file(const char * path, float scale, Adapter & ad) {
    GgufFile file(path);
    if (file.str("general.type") != "adapter" || file.str("adapter.type") != "lora") {
        set_error("the file is not a LoRA adapter GGUF (general.type=adapter, adapter.type=lora)");
        return false;
    }
    const float alpha = file.f32("adapter.lora.alpha", 0.f);
    const std::string suffix = ".lora_a";
    for (const GgufTensor & A : file.tensors()) {
        if (A.name.size() <= suffix.size() || A.name.compare(A.name.size() - suffix.size(), suffix.size(), suffix) != 0) continue;
        const std::string target = A.name.substr(0, A.name.size() - suffix.size());
        if (target == "token_embd.weight" || target.find("_exps") != std::string::npos) {
            set_error("per-row adapters refuse token-embedding and expert targets: " + target);
            return false;
        }
        const GgufTensor * B = file.find(target + ".lora_b");
        if (!B || A.ne.size() != 2 || B->ne.size() != 2 || A.ne[1] != B->ne[0] || (A.type != GGML_F32 && A.type != GGML_F16) ||
            (B->type != GGML_F32 && B->type != GGML_F16)) {
            set_error("adapter tensor pair of " + target + " is malformed");
            return false;
        }
        const uint32_t r = (uint32_t)A.ne[1];
        if (ad.rank && ad.rank != r) {
            set_error("adapter tensors disagree on their rank");
            return false;
        }
        ad.rank = r;
        auto to_f32 = [](const GgufTensor & t) {
            const size_t n = t.ne[0] * t.ne[1];
            std::vector<float> out(n);
            if (t.type == GGML_F32) {
                std::memcpy(out.data(), t.data, n * 4);
            } else {
                for (size_t i = 0; i < n; ++i) {
                    uint16_t h;
                    std::memcpy(&h, t.data + 2 * i, 2);
                    out[i] = half_to_float(h);
                }
            }
            return out;
        };
        ad.unpadded_bytes += (A.ne[0] * A.ne[1] + B->ne[0] * B->ne[1]) * 4;
        ad.ab[target] = {to_f32(A), to_f32(*B)};
    }
    if (ad.rank == 0) {
        set_error("the adapter holds no lora tensors");
        return false;
    }
    ad.scale = (alpha != 0.f ? alpha / (float)ad.rank : 1.0f) * scale;
    return true;
}

int Engine::adapter_load(const char * path, float scale, int32_t * out_id) {
    if (!path || !*path || !out_id) {
        set_error("adapter_path and out_id are required");
        return STATUS_RUNTIME;
    }
    if (!std::isfinite(scale)) {
        set_error("adapter scale must be finite");
        return STATUS_RUNTIME;
    }
    if (next_adapter_id_ == INT32_MAX) {
        set_error("per-row adapter ids are exhausted");
        return STATUS_RUNTIME;
    }
    Adapter ad;
    if (!read_adapter_file(path, scale, ad)) return STATUS_RUNTIME;
    const int32_t id = next_adapter_id_++;
    adapters_[id] = std::move(ad);
    restack_adapters();
    *out_id = id;
    return STATUS_OK;
}

// ---- one active adapter at a time (crates/retrograd-ffi/runtime/src/retro_engine.cpp:756-870). The factors live
// in the same stacks as the per-row adapters; rows with adapter == 0 are routed to the active one's index.

void Engine::forget_kv() {
    RB_CUDA(cudaStreamSynchronize(stream));
    for (uint32_t slot = 0; slot < config.n_seq_max; ++slot) kv->seq_rm((int32_t)slot, -1, -1);
    weights_version += 1;
}

int Engine::lora_load_named(const char * name, const char * path) {
    Adapter ad;
    try {
        if (!read_adapter_file(path, 1.0f, ad)) return STATUS_RUNTIME;
    } catch (const std::exception &) {
        set_error(std::string("failed to load LoRA adapter: ") + path);
        return STATUS_RUNTIME;
    }
    ad.serial = true;
    const bool was_active = active_name_ == name;
    auto found = serial_ids_.find(name);
    if (found != serial_ids_.end()) adapters_.erase(found->second);
    const int32_t id = next_adapter_id_++;
    adapters_[id] = std::move(ad);
    serial_ids_[name] = id;
    restack_adapters();
    if (was_active) {           // a reload of the active adapter re-applies it: the resident KV is stale
        active_id_ = id;
        forget_kv();
    }
    return STATUS_OK;
}

int Engine::lora_load_single(const char * path) {
    Adapter ad;
    try {
        if (!read_adapter_file(path, 1.0f, ad)) return STATUS_RUNTIME;
    } catch (const std::exception &) {
        set_error(std::string("failed to load LoRA adapter: ") + path);
        return STATUS_RUNTIME;
    }
    ad.serial = true;
    // the historical single-adapter contract: every other registered adapter goes
    for (const auto & kvp : serial_ids_) adapters_.erase(kvp.second);
    serial_ids_.clear();
    const int32_t id = next_adapter_id_++;
    adapters_[id] = std::move(ad);
    serial_ids_[path] = id;
    active_name_ = path;
    active_id_ = id;
    restack_adapters();
    forget_kv();
    return STATUS_OK;
}

int Engine::lora_activate(const char * name) {
    const std::string wanted = name ? name : "";
    int32_t id = 0;
    if (!wanted.empty()) {
        auto found = serial_ids_.find(wanted);
        if (found == serial_ids_.end()) {
            set_error("no LoRA adapter registered under '" + wanted + "'");
            return STATUS_RUNTIME;
        }
        id = found->second;
    }
    active_name_ = wanted;
    active_id_ = id;
    forget_kv();
    return STATUS_OK;
}

int Engine::lora_set_enabled(bool enabled) {
    if (!enabled) {
        active_name_.clear();
        active_id_ = 0;
    } else if (active_name_.empty()) {
        set_error("cannot enable LoRA: no adapter is active");
        return STATUS_RUNTIME;
    }
    forget_kv();        // disabling is as much a weights change as enabling
    return STATUS_OK;
}

// A frozen per-row copy of the active adapter (the trainer-owned context's policy snapshot).
int Engine::adapter_snapshot(int32_t replace, float scale, int32_t * out_id) {
    if (!out_id) {
        set_error("out_id is required");
        return STATUS_RUNTIME;
    }
    if (!std::isfinite(scale)) {
        set_error("the adapter scale must be finite");
        return STATUS_RUNTIME;
    }
    if (active_id_ == 0) {
        set_error("no trained adapter is active on the generation context: nothing to snapshot");
        return STATUS_RUNTIME;
    }
    if (replace != 0) {
        auto found = adapters_.find(replace);
        if (found == adapters_.end() || found->second.serial) {
            set_error("no per-row adapter is loaded under id " + std::to_string(replace));
            return STATUS_RUNTIME;
        }
        adapters_.erase(found);
    }
    Adapter copy = adapters_.at(active_id_);
    copy.serial = false;
    copy.scale *= scale;
    const int32_t id = next_adapter_id_++;
    adapters_[id] = std::move(copy);
    restack_adapters();
    *out_id = id;
    return STATUS_OK;
}

uint64_t Engine::work_buffer_bytes() const {
    uint64_t total = 0;
    auto add = [&](const auto & buffer) { total += (uint64_t)buffer.count * sizeof(*buffer.ptr); };
    add(block_table_); add(maps_store_); add(d_stage_); add(d_result_); add(x_); add(xn_); add(qkv_); add(att_); add(gu_); add(hff_); add(hs_);
    add(router_logits_); add(moe_w_); add(pair_gu_); add(pair_h_); add(pair_y_); add(lora_tmp_); add(logits_work_); add(logits); add(route_ids);
    add(moe_ids_); add(d_aux_); add(moe_offsets_); add(moe_sorted_); add(lora_offsets_); add(lora_sorted_); add(stream_scratch_);
    add(sample_scratch_); add(attn_scratch_); add(moe_xs_); add(moe_gu_s_); add(moe_y_s_); add(ep_all_offsets_); add(ep_offsets_l_);
    add(ep_sorted_l_); add(ep_send_); add(ep_recv_); add(ep_gu_); add(ep_h_); add(ep_y_); add(ep_back_);
    for (const SplitBuffer * sb : {&xn_split_, &att_split_, &hff_split_, &hs_split_, &moe_x_split_, &moe_h_split_}) add(sb->store);
    return total;
}

uint64_t Engine::adapter_bytes() const {
    uint64_t total = stacked_bytes_;
    for (const auto & a : adapters_) total += a.second.unpadded_bytes;      // the host copies the stacks are built from
    return total;
}

int Engine::adapter_unload(int32_t id) {
    auto found = adapters_.find(id);
    if (found == adapters_.end() || found->second.serial) {
        set_error("no per-row adapter is loaded under id " + std::to_string(id));
        return STATUS_RUNTIME;
    }
    adapters_.erase(found);
    restack_adapters();
    return STATUS_OK;
}

// Every load restacks all adapters, zero-padded to the largest rank, in F32
// (retro_lora_train.h:1298-1306).
void Engine::restack_adapters() {
    RB_CUDA(cudaStreamSynchronize(stream));
    adapter_index_.clear();
    lora_targets_.clear();
    stacked_bytes_ = 0;
    r_max_ = 0;
    const size_t n = adapters_.size();
    if (n == 0) return;
    std::vector<float> scales;
    std::map<std::string, std::pair<uint32_t, uint32_t>> shapes;   // target -> (n_in, n_out)
    for (const auto & kvp : adapters_) {
        adapter_index_[kvp.first] = (int32_t)scales.size();
        scales.push_back(kvp.second.scale);
        r_max_ = std::max(r_max_, kvp.second.rank);
        for (const auto & t : kvp.second.ab) {
            const uint32_t r = kvp.second.rank;
            shapes[t.first] = {(uint32_t)(t.second.first.size() / r), (uint32_t)(t.second.second.size() / r)};
        }
    }
    lora_scales_.ensure(n);
    RB_CUDA(cudaMemcpy(lora_scales_.ptr, scales.data(), n * 4, cudaMemcpyHostToDevice));
    for (const auto & sh : shapes) {
        auto target = std::make_unique<LoraTarget>();
        target->n_in = sh.second.first;
        target->n_out = sh.second.second;
        target->present = true;
        std::vector<float> a(n * r_max_ * target->n_in, 0.f), b(n * (size_t)target->n_out * r_max_, 0.f);
        size_t idx = 0;
        for (const auto & kvp : adapters_) {
            auto it = kvp.second.ab.find(sh.first);
            if (it != kvp.second.ab.end()) {
                const uint32_t r = kvp.second.rank;
                // A: r rows of n_in; B: n_out rows of r
                std::memcpy(&a[idx * r_max_ * target->n_in], it->second.first.data(), (size_t)r * target->n_in * 4);
                for (uint32_t o = 0; o < target->n_out; ++o)
                    std::memcpy(&b[(idx * target->n_out + o) * r_max_], &it->second.second[(size_t)o * r], r * 4);
            }
            ++idx;
        }
        target->a.ensure(a.size());
        target->b.ensure(b.size());
        RB_CUDA(cudaMemcpy(target->a.ptr, a.data(), a.size() * 4, cudaMemcpyHostToDevice));
        RB_CUDA(cudaMemcpy(target->b.ptr, b.data(), b.size() * 4, cudaMemcpyHostToDevice));
        stacked_bytes_ += (a.size() + b.size()) * 4;
        lora_targets_[sh.first] = std::move(target);
    }
    RB_CUDA(cudaDeviceSynchronize());      // the blocking uploads have reached the device before the next step's kernels
}

void Engine::adapter_info(retro_adapter_rows_info * out) {
    *out = retro_adapter_rows_info{};
    out->struct_size = sizeof(retro_adapter_rows_info);
    // the stacks also hold the registered one-at-a-time adapters; the counts describe the per-row ones
    uint32_t n = 0;
    uint64_t unpadded = 0;
    for (const auto & a : adapters_) {
        if (a.second.serial) continue;
        ++n;
        unpadded += a.second.unpadded_bytes;
    }
    out->n_adapters = n;
    out->max_rank = r_max_;
    out->stacked_bytes = stacked_bytes_;
    out->unpadded_bytes = unpadded;
}

} // namespace rb200
