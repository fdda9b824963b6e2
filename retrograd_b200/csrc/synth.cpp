// Seeded GGUF model synthesiser: writes a llama-style / qwen2-style / olmoe-style
// decoder with random weights straight into a GGUF v3 file.
//
// The container layout, tensor names, `ne` order (fastest dimension first), the
// 32-byte alignment, the metadata keys and the xorshift64* generator follow the
// reference's fixture generators (scripts/gen-tiny-fixture.py:116-133,226-374,
// scripts/gen-tiny-moe-fixture.py:192-362). The Q8_0 quantiser is the
// reference's (d = amax/127, round half away from zero; gen-tiny-fixture.py:173-198).
// The Q4_K and MXFP4 encoders are this project's own: any valid encoder will do,
// since parity is "the same bytes decoded two ways".
//
// Workloads here are synthetic by construction: weights ~ N(0, std) from the
// seeded stream, norm vectors 1 +- 0.02, no data set is involved.

#include "blocks.hpp"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace rb200 {

namespace {

struct Xorshift {
    uint64_t state;
    explicit Xorshift(uint64_t seed) : state(seed | 1) {}
    uint64_t next() {
        uint64_t s = state;
        s ^= s >> 12;
        s ^= s << 25;
        s ^= s >> 27;
        state = s;
        return s * 0x2545F4914F6CDD1DULL;
    }
    // [-1, 1) from the 24 high bits, as the reference generator draws it.
    float unit() { return (float)((double)(next() >> 40) / (double)(1 << 24) * 2.0 - 1.0); }
    // (0, 1]
    float open01() { return (float)(((next() >> 40) + 1) * (1.0 / 16777216.0)); }
};

uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}

void quantize_q8_0(const float * x, size_t n, uint8_t * out) {
    for (size_t b = 0; b < n / 32; ++b) {
        const float * v = x + b * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(v[i]));
        // The reference packs d = amax/127 computed in double and stored as f16; codes use 1/d of
        // the unrounded d.
        const double d = (double)amax / 127.0;
        const double inv = d != 0.0 ? 1.0 / d : 0.0;
        const uint16_t dh = float_to_half((float)d);
        uint8_t * o = out + b * 34;
        std::memcpy(o, &dh, 2);
        for (int i = 0; i < 32; ++i) {
            const double s = (double)v[i] * inv;
            double code = std::floor(std::fabs(s) + 0.5);
            if (code > 127.0) code = 127.0;
            o[2 + i] = (uint8_t)(int8_t)(s >= 0.0 ? (int)code : -(int)code);
        }
    }
}

void quantize_q4_k(const float * x, size_t n, uint8_t * out) {
    for (size_t b = 0; b < n / 256; ++b) {
        const float * v = x + b * 256;
        float scale[8], mneg[8];
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; ++j) {
            float lo = 0.f, hi = 0.f;
            for (int i = 0; i < 32; ++i) {
                lo = std::min(lo, v[j * 32 + i]);
                hi = std::max(hi, v[j * 32 + i]);
            }
            scale[j] = (hi - lo) / 15.f;
            mneg[j] = -lo;
            max_scale = std::max(max_scale, scale[j]);
            max_min = std::max(max_min, mneg[j]);
        }
        const uint16_t dh = float_to_half(max_scale / 63.f);
        const uint16_t mh = float_to_half(max_min / 63.f);
        const float d = half_to_float(dh), dmin = half_to_float(mh);
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) {
            int s = d > 0.f ? (int)std::lround(scale[j] / d) : 0;
            int m = dmin > 0.f ? (int)std::lround(mneg[j] / dmin) : 0;
            sc[j] = (uint8_t)std::clamp(s, 0, 63);
            mn[j] = (uint8_t)std::clamp(m, 0, 63);
        }
        uint8_t * o = out + b * 144;
        std::memcpy(o, &dh, 2);
        std::memcpy(o + 2, &mh, 2);
        uint8_t * p = o + 4;
        std::memset(p, 0, 12);
        for (int j = 0; j < 8; ++j) {
            if (j < 4) {
                p[j] |= sc[j];
                p[j + 4] |= mn[j];
            } else {
                p[j + 4] = (uint8_t)((sc[j] & 0xF) | ((mn[j] & 0xF) << 4));
                p[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
                p[j] |= (uint8_t)((mn[j] >> 4) << 6);
            }
        }
        uint8_t * qs = o + 16;
        for (int g = 0; g < 4; ++g) {
            const int j0 = 2 * g, j1 = 2 * g + 1;
            const float d0 = d * sc[j0], m0 = dmin * mn[j0];
            const float d1 = d * sc[j1], m1 = dmin * mn[j1];
            for (int i = 0; i < 32; ++i) {
                int q0 = d0 > 0.f ? (int)std::lround((v[g * 64 + i] + m0) / d0) : 0;
                int q1 = d1 > 0.f ? (int)std::lround((v[g * 64 + 32 + i] + m1) / d1) : 0;
                q0 = std::clamp(q0, 0, 15);
                q1 = std::clamp(q1, 0, 15);
                qs[g * 32 + i] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

const float kFp4Doubled[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

void quantize_mxfp4(const float * x, size_t n, uint8_t * out) {
    for (size_t b = 0; b < n / 32; ++b) {
        const float * v = x + b * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(v[i]));
        // Doubled table peaks at 12 under the half scale 2^(e-128): pick the smallest exponent
        // that keeps amax representable.
        int e = 0;
        if (amax > 0.f) {
            e = (int)std::ceil(std::log2(amax / 12.f)) + 128;
            e = std::clamp(e, 0, 254);
        }
        const float scale = e8m0_half_to_float((uint8_t)e);
        uint8_t * o = out + b * 17;
        o[0] = (uint8_t)e;
        uint8_t code[32];
        for (int i = 0; i < 32; ++i) {
            const float t = v[i] / scale;
            int best = 0;
            float err = std::fabs(t - kFp4Doubled[0]);
            for (int c = 1; c < 16; ++c) {
                if (c == 8) continue;
                const float e2 = std::fabs(t - kFp4Doubled[c]);
                if (e2 < err) { err = e2; best = c; }
            }
            code[i] = (uint8_t)best;
        }
        for (int i = 0; i < 16; ++i) o[1 + i] = (uint8_t)(code[i] | (code[i + 16] << 4));
    }
}

void encode_row(uint32_t type, const float * x, size_t n, uint8_t * out) {
    switch (type) {
        case GGML_F32: std::memcpy(out, x, n * 4); break;
        case GGML_F16:
            for (size_t i = 0; i < n; ++i) {
                const uint16_t h = float_to_half(x[i]);
                std::memcpy(out + 2 * i, &h, 2);
            }
            break;
        case GGML_Q8_0: quantize_q8_0(x, n, out); break;
        case GGML_Q4_K: quantize_q4_k(x, n, out); break;
        case GGML_MXFP4: quantize_mxfp4(x, n, out); break;
        default: throw std::runtime_error("synth: unsupported tensor type");
    }
}

uint32_t parse_type(const std::string & s) {
    if (s == "f32") return GGML_F32;
    if (s == "f16") return GGML_F16;
    if (s == "q8_0") return GGML_Q8_0;
    if (s == "q4_k" || s == "q4_K") return GGML_Q4_K;
    if (s == "mxfp4") return GGML_MXFP4;
    throw std::runtime_error("synth: unknown dtype '" + s + "'");
}

struct Spec {
    std::string arch = "llama";
    std::string name = "retrograd-b200-synth";
    uint32_t n_layer = 2, d = 256, n_head = 4, n_head_kv = 4, head_dim = 0, ff = 688, vocab = 4096;
    uint32_t n_expert = 0, n_expert_used = 0;
    uint32_t ctx_train = 8192;
    uint32_t dtype = GGML_Q8_0, expert_dtype = GGML_Q8_0, embd_dtype = 0xffffffffu;
    float std_w = 0.02f, rope_base = 10000.0f, eps = 1e-5f;
    uint64_t seed = 1;
    bool bias = false;
    // "normal": N(0, std). "uniform": std * unit().
    bool normal = true;
    // optional end-of-turn tokens: `eot` is named by tokenizer.ggml.eot_token_id and spelled <|eot_id|>;
    // `turn_end` is only spelled <|im_end|> (a control piece the loader has to recognise by its text)
    uint32_t eot = 0, turn_end = 0;
};

struct TensorPlan {
    std::string name;
    std::vector<uint64_t> ne;
    uint32_t type;
    float scale;
    float offset;
    bool vector;
    uint64_t bytes;
    uint64_t file_offset;
};

void put_u32(std::vector<uint8_t> & o, uint32_t v) { o.insert(o.end(), (uint8_t *)&v, (uint8_t *)&v + 4); }
void put_u64(std::vector<uint8_t> & o, uint64_t v) { o.insert(o.end(), (uint8_t *)&v, (uint8_t *)&v + 8); }
void put_f32(std::vector<uint8_t> & o, float v) { o.insert(o.end(), (uint8_t *)&v, (uint8_t *)&v + 4); }
void put_str(std::vector<uint8_t> & o, const std::string & s) {
    put_u64(o, s.size());
    o.insert(o.end(), s.begin(), s.end());
}
enum { T_UINT32 = 4, T_INT32 = 5, T_FLOAT32 = 6, T_BOOL = 7, T_STRING = 8, T_ARRAY = 9 };

void kv_u32(std::vector<uint8_t> & o, const std::string & k, uint32_t v) { put_str(o, k); put_u32(o, T_UINT32); put_u32(o, v); }
void kv_f32(std::vector<uint8_t> & o, const std::string & k, float v) { put_str(o, k); put_u32(o, T_FLOAT32); put_f32(o, v); }
void kv_bool(std::vector<uint8_t> & o, const std::string & k, bool v) { put_str(o, k); put_u32(o, T_BOOL); o.push_back(v ? 1 : 0); }
void kv_str(std::vector<uint8_t> & o, const std::string & k, const std::string & v) { put_str(o, k); put_u32(o, T_STRING); put_str(o, v); }

} // namespace

// Encodes one row of `n` floats as `type`; returns the bytes written, 0 when the type or the
// length is not supported.
size_t quantize_row(uint32_t type, const float * x, size_t n, uint8_t * out) {
    const size_t bytes = row_bytes(type, n);
    if (bytes == 0 || type == GGML_BF16) return 0;
    encode_row(type, x, n, out);
    return bytes;
}

// spec: whitespace-separated key=value pairs. Returns the number of bytes written.
uint64_t synth_gguf(const char * path, const char * spec_text) {
    Spec sp;
    {
        std::string text = spec_text ? spec_text : "";
        size_t pos = 0;
        while (pos < text.size()) {
            while (pos < text.size() && isspace((unsigned char)text[pos])) ++pos;
            size_t end = pos;
            while (end < text.size() && !isspace((unsigned char)text[end])) ++end;
            if (end == pos) break;
            const std::string item = text.substr(pos, end - pos);
            pos = end;
            const size_t eq = item.find('=');
            if (eq == std::string::npos) throw std::runtime_error("synth: expected key=value, got '" + item + "'");
            const std::string k = item.substr(0, eq), v = item.substr(eq + 1);
            if (k == "arch") sp.arch = v;
            else if (k == "name") sp.name = v;
            else if (k == "layers") sp.n_layer = (uint32_t)std::stoul(v);
            else if (k == "d") sp.d = (uint32_t)std::stoul(v);
            else if (k == "heads") sp.n_head = (uint32_t)std::stoul(v);
            else if (k == "kv_heads") sp.n_head_kv = (uint32_t)std::stoul(v);
            else if (k == "head_dim") sp.head_dim = (uint32_t)std::stoul(v);
            else if (k == "ff") sp.ff = (uint32_t)std::stoul(v);
            else if (k == "vocab") sp.vocab = (uint32_t)std::stoul(v);
            else if (k == "experts") sp.n_expert = (uint32_t)std::stoul(v);
            else if (k == "experts_used") sp.n_expert_used = (uint32_t)std::stoul(v);
            else if (k == "ctx_train") sp.ctx_train = (uint32_t)std::stoul(v);
            else if (k == "dtype") sp.dtype = parse_type(v);
            else if (k == "expert_dtype") sp.expert_dtype = parse_type(v);
            else if (k == "embd_dtype") sp.embd_dtype = parse_type(v);
            else if (k == "std") sp.std_w = std::stof(v);
            else if (k == "rope_base") sp.rope_base = std::stof(v);
            else if (k == "eps") sp.eps = std::stof(v);
            else if (k == "seed") sp.seed = std::stoull(v);
            else if (k == "bias") sp.bias = v == "1" || v == "true";
            else if (k == "dist") sp.normal = v != "uniform";
            else if (k == "eot") sp.eot = (uint32_t)std::stoul(v);
            else if (k == "turn_end") sp.turn_end = (uint32_t)std::stoul(v);
            else throw std::runtime_error("synth: unknown key '" + k + "'");
        }
    }
    if (sp.head_dim == 0) sp.head_dim = sp.d / sp.n_head;
    if (sp.embd_dtype == 0xffffffffu) sp.embd_dtype = sp.dtype;
    const bool moe = sp.n_expert > 0;
    if (moe && sp.arch != "olmoe") throw std::runtime_error("synth: experts need arch=olmoe");
    if (sp.n_head % sp.n_head_kv != 0) throw std::runtime_error("synth: heads must be a multiple of kv_heads");
    if (sp.vocab < 260) throw std::runtime_error("synth: vocab must hold the 259 byte-fallback tokens");

    const uint64_t dq = (uint64_t)sp.n_head * sp.head_dim, dkv = (uint64_t)sp.n_head_kv * sp.head_dim;
    std::vector<TensorPlan> plan;
    // A matrix whose row length does not divide into whole blocks is stored as F16, which is
    // what llama.cpp-style quantisers do with indivisible rows.
    auto storage = [&](uint32_t want, uint64_t row) {
        BlockGeom g{};
        block_geom(want, g);
        return row % g.elems == 0 ? want : (uint32_t)GGML_F16;
    };
    auto mat = [&](const std::string & n, std::vector<uint64_t> ne, uint32_t want) {
        plan.push_back({n, ne, storage(want, ne[0]), sp.std_w, 0.f, false, 0, 0});
    };
    auto vec = [&](const std::string & n, uint64_t len, float scale, float offset) {
        plan.push_back({n, {len}, GGML_F32, scale, offset, true, 0, 0});
    };
    mat("token_embd.weight", {sp.d, sp.vocab}, sp.embd_dtype);
    for (uint32_t l = 0; l < sp.n_layer; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        vec(p + "attn_norm.weight", sp.d, 0.02f, 1.0f);
        mat(p + "attn_q.weight", {sp.d, dq}, sp.dtype);
        if (sp.bias) vec(p + "attn_q.bias", dq, 0.01f, 0.f);
        mat(p + "attn_k.weight", {sp.d, dkv}, sp.dtype);
        if (sp.bias) vec(p + "attn_k.bias", dkv, 0.01f, 0.f);
        mat(p + "attn_v.weight", {sp.d, dkv}, sp.dtype);
        if (sp.bias) vec(p + "attn_v.bias", dkv, 0.01f, 0.f);
        if (sp.arch == "olmoe") {
            vec(p + "attn_q_norm.weight", dq, 0.02f, 1.0f);
            vec(p + "attn_k_norm.weight", dkv, 0.02f, 1.0f);
        }
        mat(p + "attn_output.weight", {dq, sp.d}, sp.dtype);
        vec(p + "ffn_norm.weight", sp.d, 0.02f, 1.0f);
        if (moe) {
            plan.push_back({p + "ffn_gate_inp.weight", {sp.d, sp.n_expert}, GGML_F32, sp.std_w * 4.f, 0.f, false, 0, 0});
            mat(p + "ffn_gate_exps.weight", {sp.d, sp.ff, sp.n_expert}, sp.expert_dtype);
            mat(p + "ffn_up_exps.weight", {sp.d, sp.ff, sp.n_expert}, sp.expert_dtype);
            mat(p + "ffn_down_exps.weight", {sp.ff, sp.d, sp.n_expert}, sp.expert_dtype);
        } else {
            mat(p + "ffn_gate.weight", {sp.d, sp.ff}, sp.dtype);
            mat(p + "ffn_up.weight", {sp.d, sp.ff}, sp.dtype);
            mat(p + "ffn_down.weight", {sp.ff, sp.d}, sp.dtype);
        }
    }
    vec("output_norm.weight", sp.d, 0.02f, 1.0f);
    mat("output.weight", {sp.d, sp.vocab}, sp.dtype);
    if (sp.bias) vec("output.bias", sp.vocab, 0.01f, 0.f);

    uint64_t offset = 0;
    for (auto & t : plan) {
        uint64_t rows = 1;
        for (size_t i = 1; i < t.ne.size(); ++i) rows *= t.ne[i];
        t.bytes = row_bytes(t.type, t.ne[0]) * rows;
        t.file_offset = offset;
        offset += (t.bytes + 31) / 32 * 32;
    }

    std::vector<uint8_t> h;
    std::vector<uint8_t> kvs;
    uint64_t n_kv = 0;
    const std::string a = sp.arch;
    kv_str(kvs, "general.architecture", a); ++n_kv;
    kv_str(kvs, "general.name", sp.name); ++n_kv;
    kv_u32(kvs, a + ".block_count", sp.n_layer); ++n_kv;
    kv_u32(kvs, a + ".context_length", sp.ctx_train); ++n_kv;
    kv_u32(kvs, a + ".embedding_length", sp.d); ++n_kv;
    kv_u32(kvs, a + ".feed_forward_length", sp.ff); ++n_kv;
    kv_u32(kvs, a + ".attention.head_count", sp.n_head); ++n_kv;
    kv_u32(kvs, a + ".attention.head_count_kv", sp.n_head_kv); ++n_kv;
    kv_u32(kvs, a + ".attention.key_length", sp.head_dim); ++n_kv;
    kv_u32(kvs, a + ".attention.value_length", sp.head_dim); ++n_kv;
    kv_f32(kvs, a + ".attention.layer_norm_rms_epsilon", sp.eps); ++n_kv;
    kv_u32(kvs, a + ".rope.dimension_count", sp.head_dim); ++n_kv;
    kv_f32(kvs, a + ".rope.freq_base", sp.rope_base); ++n_kv;
    kv_u32(kvs, a + ".vocab_size", sp.vocab); ++n_kv;
    if (moe) {
        kv_u32(kvs, a + ".expert_count", sp.n_expert); ++n_kv;
        kv_u32(kvs, a + ".expert_used_count", sp.n_expert_used); ++n_kv;
    }
    kv_str(kvs, "tokenizer.ggml.model", "llama"); ++n_kv;
    {
        // Byte-fallback vocabulary: three specials, the 256 bytes, then ordinary filler pieces.
        put_str(kvs, "tokenizer.ggml.tokens"); put_u32(kvs, T_ARRAY); put_u32(kvs, T_STRING); put_u64(kvs, sp.vocab);
        std::vector<int32_t> types(sp.vocab, 1);
        for (uint32_t i = 0; i < sp.vocab; ++i) {
            std::string tok;
            if (i == 0) { tok = "<unk>"; types[i] = 2; }
            else if (i == 1) { tok = "<s>"; types[i] = 3; }
            else if (i == 2) { tok = "</s>"; types[i] = 3; }
            else if (i < 259) {
                char buf[8];
                std::snprintf(buf, sizeof buf, "<0x%02X>", i - 3);
                tok = buf;
                types[i] = 6;
            } else if (sp.eot && i == sp.eot) {
                tok = "<|eot_id|>";
                types[i] = 3;
            } else if (sp.turn_end && i == sp.turn_end) {
                tok = "<|im_end|>";
                types[i] = 3;
            } else {
                tok = "\xE2\x96\x81t" + std::to_string(i);
            }
            put_str(kvs, tok);
        }
        ++n_kv;
        put_str(kvs, "tokenizer.ggml.scores"); put_u32(kvs, T_ARRAY); put_u32(kvs, T_FLOAT32); put_u64(kvs, sp.vocab);
        for (uint32_t i = 0; i < sp.vocab; ++i) put_f32(kvs, 0.f);
        ++n_kv;
        put_str(kvs, "tokenizer.ggml.token_type"); put_u32(kvs, T_ARRAY); put_u32(kvs, T_INT32); put_u64(kvs, sp.vocab);
        for (uint32_t i = 0; i < sp.vocab; ++i) put_u32(kvs, (uint32_t)types[i]);
        ++n_kv;
    }
    kv_u32(kvs, "tokenizer.ggml.bos_token_id", 1); ++n_kv;
    kv_u32(kvs, "tokenizer.ggml.eos_token_id", 2); ++n_kv;
    kv_u32(kvs, "tokenizer.ggml.unknown_token_id", 0); ++n_kv;
    if (sp.eot) { kv_u32(kvs, "tokenizer.ggml.eot_token_id", sp.eot); ++n_kv; }
    kv_bool(kvs, "tokenizer.ggml.add_bos_token", true); ++n_kv;
    kv_bool(kvs, "tokenizer.ggml.add_eos_token", false); ++n_kv;
    kv_u32(kvs, "general.alignment", 32); ++n_kv;

    put_u32(h, 0x46554747u);
    put_u32(h, 3);
    put_u64(h, plan.size());
    put_u64(h, n_kv);
    h.insert(h.end(), kvs.begin(), kvs.end());
    for (auto & t : plan) {
        put_str(h, t.name);
        put_u32(h, (uint32_t)t.ne.size());
        for (uint64_t dim : t.ne) put_u64(h, dim);
        put_u32(h, t.type);
        put_u64(h, t.file_offset);
    }
    while (h.size() % 32) h.push_back(0);

    FILE * f = std::fopen(path, "wb");
    if (!f) throw std::runtime_error(std::string("synth: cannot open ") + path);
    if (std::fwrite(h.data(), 1, h.size(), f) != h.size()) { std::fclose(f); throw std::runtime_error("synth: short write"); }
    uint64_t written = h.size();

    std::vector<uint8_t> buf;
    for (size_t ti = 0; ti < plan.size(); ++ti) {
        const TensorPlan & t = plan[ti];
        uint64_t rows = 1;
        for (size_t i = 1; i < t.ne.size(); ++i) rows *= t.ne[i];
        const uint64_t n = t.ne[0];
        const size_t rb = row_bytes(t.type, n);
        const uint64_t padded = (t.bytes + 31) / 32 * 32;
        buf.assign(padded, 0);
        const uint64_t tseed = mix64(sp.seed * 0x100000001B3ULL + ti);
        const bool normal = sp.normal && !t.vector;
#pragma omp parallel
        {
            std::vector<float> row(n);
#pragma omp for schedule(static)
            for (int64_t r = 0; r < (int64_t)rows; ++r) {
                Xorshift rng(mix64(tseed ^ (uint64_t)r * 0xD1B54A32D192ED03ULL));
                if (normal) {
                    for (uint64_t i = 0; i < n; i += 2) {
                        const float u1 = rng.open01(), u2 = rng.open01();
                        const float rad = std::sqrt(-2.0f * std::log(u1));
                        const float ang = 6.28318530717958647692f * u2;
                        row[i] = t.offset + t.scale * rad * std::cos(ang);
                        if (i + 1 < n) row[i + 1] = t.offset + t.scale * rad * std::sin(ang);
                    }
                } else {
                    for (uint64_t i = 0; i < n; ++i) row[i] = t.offset + t.scale * rng.unit();
                }
                encode_row(t.type, row.data(), n, buf.data() + (size_t)r * rb);
            }
        }
        if (std::fwrite(buf.data(), 1, padded, f) != padded) { std::fclose(f); throw std::runtime_error("synth: short write"); }
        written += padded;
    }
    std::fclose(f);
    return written;
}

} // namespace rb200
