// TEST INFRASTRUCTURE - CPU restatement ("oracle") of the reference's batched decode step.
//
// Nothing here ships: only the test suite, the smoke check and the CPU-baseline leg of the
// benchmark may load this library. The product path never calls it.
//
// PARITY STATUS: the arithmetic of the reference's decode step lives in an un-vendored
// third-party dependency (the llama.cpp fork `tterrasson/llama.cpp-retrograd`, branch
// `retrograd/main`, upstream base ggml-org/llama.cpp @ cd8427d018c07eefab6c110f7f115c31ec4c6157,
// crates/retrograd-ffi/runtime/llama.cpp.lock:6-7) and the reference's own tests store no expected
// tokens or logits for a generation. The forward pass below is therefore "parity unpinned" at
// that boundary. What IS pinned against in-tree reference artefacts (see tests/golden):
//   - block decoders            crates/rir-core/src/quant.rs:82-129,223-299,399-417 (+ KATs :533-581)
//   - dequant GEMV, f32 serial  generated/rir/mul_mat_vec_q4_K/cpu.rs:52-121, mul_mat_vec_q8_0/cpu.rs:52-81
//   - RMSNorm formula           generated/rir/rms_norm/kernel.shared_reduce.cu:43-56
//   - GGUF container + Q8_0 enc scripts/gen-tiny-fixture.py:173-198,343-374 (SHA-256 of fixtures)
//   - sampling / logprob / topk crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:41-51,103-225,718-875,2942-2985
//   - step batch order          crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:2572-2603
//   - MoE routing known-answer  tests/expert_placement.rs:379-425
//
// Conventions fixed here because the fork is absent: RoPE pairs are adjacent for
// general.architecture=llama and half-split for qwen2/olmoe; GQA maps q head h to kv head
// h / (Hq/Hkv); attention scale 1/sqrt(head_dim); causal mask by position within the slot; K/V
// are rounded to f16 when stored (or, for a context of kv_dtype Q8_0 / Q4_0, pass through ggml's row quantisers);
// activations stay f32 (the in-tree GEMV oracles' semantics, "act = f32": what parity is stated against). The
// optional "act = q8" mode re-quantises activations in the weight matmuls the way the reference's CPU backend does
// (tests/lora_rows.rs:16-20); it restates published ggml routines, is pinned by nothing in the reference's tree, and
// is only ever reported beside act = f32.

#include <omp.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <numeric>
#include <random>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

thread_local std::string g_error;

// ---------------------------------------------------------------------------------------------
// Scalar formats (crates/rir-core/src/quant.rs:82-129)

float half_to_f32(uint16_t h) {
    const uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, mant = h & 0x3ff;
    uint32_t bits;
    if (exp == 0 && mant == 0) {
        bits = sign << 31;
    } else if (exp == 0) {
        int e = -1;
        uint32_t m = mant;
        while ((m & 0x400) == 0) { m <<= 1; e -= 1; }
        m &= 0x3ff;
        bits = (sign << 31) | ((uint32_t)(127 - 13 + e) << 23) | (m << 13);
    } else if (exp == 0x1f) {
        bits = (sign << 31) | (0xffu << 23) | (mant << 13);
    } else {
        bits = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// Nearest-even f32 -> f16 -> f32: what storing a KV cell as F16 does to a value.
float round_to_half(float v) {
    uint32_t x;
    std::memcpy(&x, &v, 4);
    const uint32_t sign = x & 0x80000000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return v;
    if (x >= 0x477ff000u) {
        uint32_t inf = sign | 0x7f800000u;
        float f;
        std::memcpy(&f, &inf, 4);
        return f;
    }
    float a;
    std::memcpy(&a, &x, 4);
    if (x < 0x38800000u) {
        // subnormal half: quantum 2^-24
        const float q = std::nearbyintf(a * 16777216.0f) / 16777216.0f;
        return sign ? -q : q;
    }
    const uint32_t rem = x & 0x1fffu;
    x &= ~0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (x & 0x2000u))) x += 0x2000u;
    x |= sign;
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

float e8m0_to_f32_half(uint8_t x) {
    const uint32_t bits = x == 0 ? 0x00200000u : x == 1 ? 0x00400000u : ((uint32_t)x - 1) << 23;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

const int8_t KVALUES_FP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

void scale_min_k4(int j, const uint8_t * q, uint8_t & sc, uint8_t & m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

enum : uint32_t { T_F32 = 0, T_F16 = 1, T_Q8_0 = 8, T_Q4_K = 12, T_BF16 = 30, T_MXFP4 = 39 };

bool geom(uint32_t type, size_t & elems, size_t & bytes) {
    switch (type) {
        case T_F32: elems = 1; bytes = 4; return true;
        case T_F16: elems = 1; bytes = 2; return true;
        case T_BF16: elems = 1; bytes = 2; return true;
        case T_Q8_0: elems = 32; bytes = 34; return true;
        case T_Q4_K: elems = 256; bytes = 144; return true;
        case T_MXFP4: elems = 32; bytes = 17; return true;
        default: return false;
    }
}

// Block decoders (crates/rir-core/src/quant.rs:223-299,399-417).
bool dequantize_row(uint32_t type, const uint8_t * src, size_t n, float * y) {
    size_t be, bb;
    if (!geom(type, be, bb) || n % be != 0) return false;
    const size_t nb = n / be;
    switch (type) {
        case T_F32:
            std::memcpy(y, src, n * 4);
            return true;
        case T_F16:
            for (size_t i = 0; i < n; ++i) {
                uint16_t h;
                std::memcpy(&h, src + 2 * i, 2);
                y[i] = half_to_f32(h);
            }
            return true;
        case T_BF16:
            for (size_t i = 0; i < n; ++i) {
                uint16_t h;
                std::memcpy(&h, src + 2 * i, 2);
                uint32_t bits = (uint32_t)h << 16;
                std::memcpy(&y[i], &bits, 4);
            }
            return true;
        case T_Q8_0:
            for (size_t b = 0; b < nb; ++b) {
                const uint8_t * p = src + b * 34;
                uint16_t h;
                std::memcpy(&h, p, 2);
                const float scale = half_to_f32(h);
                for (int j = 0; j < 32; ++j) y[b * 32 + j] = scale * (float)(int8_t)p[2 + j];
            }
            return true;
        case T_MXFP4:
            for (size_t b = 0; b < nb; ++b) {
                const uint8_t * p = src + b * 17;
                const float scale = e8m0_to_f32_half(p[0]);
                for (int j = 0; j < 16; ++j) {
                    const uint8_t q = p[1 + j];
                    y[b * 32 + j] = scale * (float)KVALUES_FP4[q & 0x0F];
                    y[b * 32 + j + 16] = scale * (float)KVALUES_FP4[q >> 4];
                }
            }
            return true;
        case T_Q4_K:
            for (size_t b = 0; b < nb; ++b) {
                const uint8_t * p = src + b * 144;
                uint16_t h0, h1;
                std::memcpy(&h0, p, 2);
                std::memcpy(&h1, p + 2, 2);
                const float d = half_to_f32(h0), dmin = half_to_f32(h1);
                const uint8_t * scales = p + 4;
                const uint8_t * qs = p + 16;
                float * o = y + b * 256;
                for (int blk = 0, is = 0; blk < 256; blk += 64, is += 2) {
                    const uint8_t * q = qs + blk / 2;
                    uint8_t sc1, m1, sc2, m2;
                    scale_min_k4(is, scales, sc1, m1);
                    scale_min_k4(is + 1, scales, sc2, m2);
                    const float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
                    const float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
                    for (int l = 0; l < 32; ++l) {
                        o[blk + l] = d1 * (float)(q[l] & 0xF) - mm1;
                        o[blk + 32 + l] = d2 * (float)(q[l] >> 4) - mm2;
                    }
                }
            }
            return true;
    }
    return false;
}

// ---------------------------------------------------------------------------------------------
// GGUF v3 reader (layout as written by scripts/gen-tiny-fixture.py:343-374).

struct Tensor {
    std::string name;
    std::vector<uint64_t> ne;
    uint32_t type = 0;
    const uint8_t * data = nullptr;
    size_t rows() const {
        size_t r = 1;
        for (size_t i = 1; i < ne.size(); ++i) r *= ne[i];
        return r;
    }
    size_t row_bytes() const {
        size_t be, bb;
        geom(type, be, bb);
        return ne[0] / be * bb;
    }
};

struct Gguf {
    int fd = -1;
    const uint8_t * base = nullptr;
    size_t size = 0;
    std::map<std::string, uint32_t> u32;
    std::map<std::string, float> f32;
    std::map<std::string, std::string> str;
    std::map<std::string, uint64_t> arr_len;
    std::map<std::string, Tensor> tensors;
    ~Gguf() {
        if (base) munmap((void *)base, size);
        if (fd >= 0) close(fd);
    }
};

struct Cursor {
    const uint8_t * p;
    const uint8_t * end;
    template <class T> T get() {
        if (p + sizeof(T) > end) throw std::runtime_error("gguf: truncated");
        T v;
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (p + n > end) throw std::runtime_error("gguf: truncated string");
        std::string s((const char *)p, n);
        p += n;
        return s;
    }
};

size_t scalar_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: throw std::runtime_error("gguf: unknown value type");
    }
}

std::unique_ptr<Gguf> gguf_open(const char * path) {
    auto g = std::make_unique<Gguf>();
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) throw std::runtime_error(std::string("cannot open ") + path);
    struct stat st;
    fstat(g->fd, &st);
    g->size = st.st_size;
    g->base = (const uint8_t *)mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (g->base == MAP_FAILED) { g->base = nullptr; throw std::runtime_error("mmap failed"); }
    Cursor c{g->base, g->base + g->size};
    if (c.get<uint32_t>() != 0x46554747u) throw std::runtime_error("gguf: bad magic");
    if (c.get<uint32_t>() != 3) throw std::runtime_error("gguf: unsupported version");
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    uint32_t alignment = 32;
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t t = c.get<uint32_t>();
        if (t == 8) {
            g->str[key] = c.str();
        } else if (t == 9) {
            const uint32_t et = c.get<uint32_t>();
            const uint64_t n = c.get<uint64_t>();
            g->arr_len[key] = n;
            if (et == 8) {
                for (uint64_t j = 0; j < n; ++j) c.str();
            } else {
                c.p += scalar_size(et) * n;
            }
        } else if (t == 4 || t == 5) {
            g->u32[key] = c.get<uint32_t>();
        } else if (t == 6) {
            g->f32[key] = c.get<float>();
        } else {
            c.p += scalar_size(t);
        }
    }
    if (g->u32.count("general.alignment")) alignment = g->u32["general.alignment"];
    std::vector<std::pair<std::string, uint64_t>> offsets;
    for (uint64_t i = 0; i < n_tensors; ++i) {
        Tensor t;
        t.name = c.str();
        const uint32_t nd = c.get<uint32_t>();
        for (uint32_t d = 0; d < nd; ++d) t.ne.push_back(c.get<uint64_t>());
        t.type = c.get<uint32_t>();
        offsets.emplace_back(t.name, c.get<uint64_t>());
        g->tensors[t.name] = t;
    }
    size_t data_start = (size_t)(c.p - g->base);
    data_start = (data_start + alignment - 1) / alignment * alignment;
    for (auto & o : offsets) {
        Tensor & t = g->tensors[o.first];
        size_t be, bb;
        if (!geom(t.type, be, bb)) throw std::runtime_error("gguf: tensor " + t.name + " has an unsupported type");
        t.data = g->base + data_start + o.second;
        if (t.data + t.row_bytes() * t.rows() > g->base + g->size) throw std::runtime_error("gguf: tensor data out of range");
    }
    return g;
}

// ---------------------------------------------------------------------------------------------
// Model + forward

struct Lora {
    float scale = 1.f;  // alpha / rank * user scale
    uint32_t rank = 0;
    // target tensor name -> (A [in, r] stored r rows of in; B [r, out] stored out rows of r)
    std::map<std::string, std::pair<std::vector<float>, std::vector<float>>> ab;
};

struct Model {
    std::unique_ptr<Gguf> g;
    std::string arch;
    uint32_t n_layer = 0, d = 0, n_head = 0, n_head_kv = 0, head_dim = 0, ff = 0, vocab = 0;
    uint32_t n_expert = 0, n_expert_used = 0, n_rot = 0;
    float eps = 1e-5f, rope_base = 10000.f;
    bool neox = false;
    bool fast = false;  // vectorisable accumulation for timing runs; parity runs keep serial order
    // act = q8: the weight matmuls re-quantise every activation row to the 8-bit block format the weight type's dot
    // product takes and multiply integers, as the reference's CPU backend does ("the quantized base re-quantizes every
    // activation it reads", tests/lora_rows.rs:16-20). Default act = f32: the in-tree RIR oracles' semantics, which is
    // what every parity claim of this project is made against.
    bool act_q8 = false;
    std::map<int32_t, Lora> loras;
    int32_t next_lora = 1;
    std::vector<float> inv_freq;
    const Tensor * find(const std::string & n) const {
        auto it = g->tensors.find(n);
        return it == g->tensors.end() ? nullptr : &it->second;
    }
    const Tensor & need(const std::string & n) const {
        const Tensor * t = find(n);
        if (!t) throw std::runtime_error("model is missing tensor " + n);
        return *t;
    }
};

// ---- act = q8: ggml's CPU dot products over re-quantised activations. The library is absent with the un-vendored
// llama.cpp fork; these restate its published reference routines (quantize_row_q8_0_ref, quantize_row_q8_K_ref,
// ggml_vec_dot_q8_0_q8_0, ggml_vec_dot_q4_K_q8_K, ggml_vec_dot_mxfp4_q8_0 and the f16 dot for F16 weights, generic
// forms) and are pinned by nothing here: PARITY UNPINNED, reported beside act = f32 results, never as the checker.
struct ActQ80 { std::vector<float> d; std::vector<int8_t> q; };          // per 32 elements: f16-rounded scale, 32 quants
struct ActQ8K { std::vector<float> d; std::vector<int8_t> q; std::vector<int16_t> bsums; };   // per 256: scale, quants, sums of 16

void quantize_act_q8_0(const float * x, size_t n, ActQ80 & a) {
    a.d.resize(n / 32);
    a.q.resize(n);
    for (size_t b = 0; b < n / 32; ++b) {
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = std::max(amax, std::fabs(x[b * 32 + j]));
        const float d = amax / 127.f, id = d != 0.f ? 1.0f / d : 0.f;
        a.d[b] = round_to_half(d);
        for (int j = 0; j < 32; ++j) a.q[b * 32 + j] = (int8_t)std::lround(x[b * 32 + j] * id);
    }
}

void quantize_act_q8_K(const float * x, size_t n, ActQ8K & a) {
    a.d.resize(n / 256);
    a.q.resize(n);
    a.bsums.assign(n / 16, 0);
    for (size_t b = 0; b < n / 256; ++b) {
        float amax = 0.f, mx = 0.f;
        for (int j = 0; j < 256; ++j) {
            const float ax = std::fabs(x[b * 256 + j]);
            if (ax > amax) { amax = ax; mx = x[b * 256 + j]; }
        }
        if (amax == 0.f) {
            a.d[b] = 0.f;
            for (int j = 0; j < 256; ++j) a.q[b * 256 + j] = 0;
            continue;
        }
        const float iscale = -127.f / mx;
        for (int j = 0; j < 256; ++j) {
            const int v = (int)std::nearbyintf(iscale * x[b * 256 + j]);       // round to nearest, ties to even
            a.q[b * 256 + j] = (int8_t)std::min(127, v);
        }
        for (int j = 0; j < 16; ++j) {
            int sum = 0;
            for (int i = 0; i < 16; ++i) sum += a.q[b * 256 + j * 16 + i];
            a.bsums[b * 16 + j] = (int16_t)sum;
        }
        a.d[b] = 1.0f / iscale;
    }
}

float dot_q8_0_q8_0(const uint8_t * w, const ActQ80 & a, size_t n) {
    float sumf = 0.f;
    for (size_t b = 0; b < n / 32; ++b) {
        const uint8_t * p = w + b * 34;
        uint16_t h;
        std::memcpy(&h, p, 2);
        int sumi = 0;
        for (int j = 0; j < 32; ++j) sumi += (int)(int8_t)p[2 + j] * (int)a.q[b * 32 + j];
        sumf += (float)sumi * (half_to_f32(h) * a.d[b]);
    }
    return sumf;
}

float dot_mxfp4_q8_0(const uint8_t * w, const ActQ80 & a, size_t n) {
    float sumf = 0.f;
    for (size_t b = 0; b < n / 32; ++b) {
        const uint8_t * p = w + b * 17;
        const float d = a.d[b] * e8m0_to_f32_half(p[0]);
        int sumi = 0;
        for (int j = 0; j < 16; ++j) {
            sumi += (int)a.q[b * 32 + j] * KVALUES_FP4[p[1 + j] & 0x0F];
            sumi += (int)a.q[b * 32 + j + 16] * KVALUES_FP4[p[1 + j] >> 4];
        }
        sumf += d * (float)sumi;
    }
    return sumf;
}

float dot_q4_K_q8_K(const uint8_t * w, const ActQ8K & a, size_t n) {
    float sumf = 0.f;
    for (size_t b = 0; b < n / 256; ++b) {
        const uint8_t * p = w + b * 144;
        uint16_t h0, h1;
        std::memcpy(&h0, p, 2);
        std::memcpy(&h1, p + 2, 2);
        const float d = a.d[b] * half_to_f32(h0), dmin = a.d[b] * half_to_f32(h1);
        const uint8_t * scales = p + 4, * qs = p + 16;
        const int8_t * q8 = a.q.data() + b * 256;
        int sum_main = 0, sum_min = 0;
        for (int g = 0; g < 4; ++g) {
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(2 * g, scales, sc1, m1);
            scale_min_k4(2 * g + 1, scales, sc2, m2);
            int lo = 0, hi = 0;
            for (int l = 0; l < 32; ++l) {
                lo += (int)(qs[g * 32 + l] & 0xF) * (int)q8[g * 64 + l];
                hi += (int)(qs[g * 32 + l] >> 4) * (int)q8[g * 64 + 32 + l];
            }
            sum_main += (int)sc1 * lo + (int)sc2 * hi;
            sum_min += (int)m1 * ((int)a.bsums[b * 16 + 4 * g] + (int)a.bsums[b * 16 + 4 * g + 1]) +
                       (int)m2 * ((int)a.bsums[b * 16 + 4 * g + 2] + (int)a.bsums[b * 16 + 4 * g + 3]);
        }
        sumf += d * (float)sum_main - dmin * (float)sum_min;
    }
    return sumf;
}

bool act_q8_applies(uint32_t type, size_t n_in) {
    return ((type == T_Q8_0 || type == T_MXFP4) && n_in % 32 == 0) || (type == T_Q4_K && n_in % 256 == 0) || type == T_F16;
}

// Y = X W^T with the activations in the weight type's 8-bit (F16 weights: 16-bit) dot format
void matmul_act_q8(const Tensor & w, const uint8_t * wdata, size_t n_out, const float * x, size_t T, size_t n_in, float * y, size_t y_stride) {
    const size_t rb = w.row_bytes();
    std::vector<ActQ80> a80(w.type == T_Q8_0 || w.type == T_MXFP4 ? T : 0);
    std::vector<ActQ8K> a8k(w.type == T_Q4_K ? T : 0);
    std::vector<float> xh(w.type == T_F16 ? T * n_in : 0);
    for (size_t t = 0; t < T; ++t) {
        if (!a80.empty()) quantize_act_q8_0(x + t * n_in, n_in, a80[t]);
        if (!a8k.empty()) quantize_act_q8_K(x + t * n_in, n_in, a8k[t]);
        if (!xh.empty())
            for (size_t i = 0; i < n_in; ++i) xh[t * n_in + i] = round_to_half(x[t * n_in + i]);
    }
#pragma omp parallel
    {
        std::vector<float> row(w.type == T_F16 ? n_in : 0);
#pragma omp for schedule(static)
        for (int64_t o = 0; o < (int64_t)n_out; ++o) {
            const uint8_t * wr = wdata + (size_t)o * rb;
            if (w.type == T_F16) dequantize_row(w.type, wr, n_in, row.data());
            for (size_t t = 0; t < T; ++t) {
                float acc = 0.f;
                if (w.type == T_Q8_0) acc = dot_q8_0_q8_0(wr, a80[t], n_in);
                else if (w.type == T_MXFP4) acc = dot_mxfp4_q8_0(wr, a80[t], n_in);
                else if (w.type == T_Q4_K) acc = dot_q4_K_q8_K(wr, a8k[t], n_in);
                else
                    for (size_t i = 0; i < n_in; ++i) acc += row[i] * xh[t * n_in + i];
                y[t * y_stride + o] = acc;
            }
        }
    }
}

// Y[t][o] = sum_i deq(W)[o][i] * X[t][i], f32, columns in serial order
// (generated/rir/mul_mat_vec_q4_K/cpu.rs:52-121).
void matmul(const Model & m, const Tensor & w, const uint8_t * wdata, size_t n_out, const float * x, size_t T, size_t n_in,
            float * y, size_t y_stride) {
    if (m.act_q8 && act_q8_applies(w.type, n_in)) {
        matmul_act_q8(w, wdata, n_out, x, T, n_in, y, y_stride);
        return;
    }
    const size_t rb = w.row_bytes();
#pragma omp parallel
    {
        std::vector<float> row(n_in);
#pragma omp for schedule(static)
        for (int64_t o = 0; o < (int64_t)n_out; ++o) {
            dequantize_row(w.type, wdata + (size_t)o * rb, n_in, row.data());
            for (size_t t = 0; t < T; ++t) {
                const float * xv = x + t * n_in;
                float acc = 0.f;
                if (m.fast) {
#pragma omp simd reduction(+ : acc)
                    for (size_t i = 0; i < n_in; ++i) acc += row[i] * xv[i];
                } else {
                    for (size_t i = 0; i < n_in; ++i) acc += row[i] * xv[i];
                }
                y[t * y_stride + o] = acc;
            }
        }
    }
}

void rms_norm(const float * x, const float * w, size_t n, float eps, float * y) {
    // generated/rir/rms_norm/kernel.shared_reduce.cu:43-56: y = x * 1/sqrt(mean(x^2) + eps), then * w
    float ss = 0.f;
    for (size_t i = 0; i < n; ++i) ss += x[i] * x[i];
    const float scale = 1.0f / std::sqrt(ss / (float)n + eps);
    for (size_t i = 0; i < n; ++i) y[i] = x[i] * scale * w[i];
}

struct SlotKV {
    int32_t pos_min = -1, pos_max = -1;
    // [layer][pos * dkv]
    std::vector<std::vector<float>> k, v;
};

struct Ctx {
    Model * m;
    uint32_t n_slots, n_ctx_seq;
    int kv_dtype;      // retro_engine_kv_dtype: 0 F32, 1 F16, 2 Q8_0, 3 Q4_0 - what a stored K / V row is rounded to
    std::vector<SlotKV> slots;
    // filled by the last step when the model is MoE: [layer][token][k] expert ids
    std::vector<int32_t> last_routes;
    std::vector<float> last_route_margins;      // per (layer, token): the smallest probability gap that decided the selection or its order
};

const float * vec_f32(const Model & m, const std::string & name) {
    const Tensor & t = m.need(name);
    if (t.type != T_F32) throw std::runtime_error(name + " must be F32");
    return (const float *)t.data;
}

// What the cache returns for a row stored under `kv_dtype`. The quantised types are ggml's block formats over 32
// consecutive elements (published reference quantisers quantize_row_q8_0_ref / quantize_row_q4_0_ref of the
// un-vendored llama.cpp fork, restated; the reference hands the type to that library at
// crates/retrograd-ffi/runtime/src/retro_engine.cpp:84-90,251-266): the scale is kept as f16, a value reads back as
// scale * quant in f32. Q8_0: d = amax / 127, q = round-half-away(x / d). Q4_0: d = (the element of largest
// magnitude, the first of equals) / -8, q = min(15, trunc(x / d + 8.5)), value (q - 8) * d.
void kv_store_row(int kv_dtype, const float * src, float * dst, size_t n) {
    if (kv_dtype == 0) {
        std::copy(src, src + n, dst);
    } else if (kv_dtype == 1) {
        for (size_t i = 0; i < n; ++i) dst[i] = round_to_half(src[i]);
    } else if (kv_dtype == 2) {
        for (size_t b = 0; b + 32 <= n; b += 32) {
            float amax = 0.f;
            for (int j = 0; j < 32; ++j) amax = std::max(amax, std::fabs(src[b + j]));
            const float d = amax / 127.f, id = d != 0.f ? 1.0f / d : 0.f, dh = round_to_half(d);
            for (int j = 0; j < 32; ++j) dst[b + j] = dh * (float)(int8_t)std::lround(src[b + j] * id);
        }
    } else {
        for (size_t b = 0; b + 32 <= n; b += 32) {
            float amax = 0.f, mx = 0.f;
            for (int j = 0; j < 32; ++j)
                if (amax < std::fabs(src[b + j])) { amax = std::fabs(src[b + j]); mx = src[b + j]; }
            const float d = mx / -8.f, id = d != 0.f ? 1.0f / d : 0.f, dh = round_to_half(d);
            for (int j = 0; j < 32; ++j) {
                const int q = std::min(15, (int)(int8_t)(src[b + j] * id + 8.5f));
                dst[b + j] = dh * (float)(q - 8);
            }
        }
    }
}

void rope(float * v, uint32_t n_heads, uint32_t hd, uint32_t n_rot, bool neox, int32_t pos, const std::vector<float> & inv_freq) {
    for (uint32_t h = 0; h < n_heads; ++h) {
        float * p = v + (size_t)h * hd;
        for (uint32_t i = 0; i < n_rot / 2; ++i) {
            const float theta = (float)pos * inv_freq[i];
            const float c = std::cos(theta), s = std::sin(theta);
            const uint32_t i0 = neox ? i : 2 * i, i1 = neox ? i + n_rot / 2 : 2 * i + 1;
            const float a = p[i0], b = p[i1];
            p[i0] = a * c - b * s;
            p[i1] = a * s + b * c;
        }
    }
}

void apply_lora(const Model & m, int32_t adapter, const std::string & target, const float * x, size_t n_in, float * y, size_t n_out) {
    if (adapter <= 0) return;
    auto it = m.loras.find(adapter);
    if (it == m.loras.end()) return;
    auto ab = it->second.ab.find(target);
    if (ab == it->second.ab.end()) return;
    const uint32_t r = it->second.rank;
    const std::vector<float> & A = ab->second.first;
    const std::vector<float> & B = ab->second.second;
    std::vector<float> t(r, 0.f);
    for (uint32_t j = 0; j < r; ++j) {
        float acc = 0.f;
        for (size_t i = 0; i < n_in; ++i) acc += A[(size_t)j * n_in + i] * x[i];
        t[j] = acc;
    }
    for (size_t o = 0; o < n_out; ++o) {
        float acc = 0.f;
        for (uint32_t j = 0; j < r; ++j) acc += B[o * r + j] * t[j];
        y[o] += it->second.scale * acc;
    }
}

void linear(const Model & m, const std::string & name, const float * x, size_t T, size_t n_in, float * y, size_t n_out,
            const int32_t * adapters) {
    const Tensor & w = m.need(name + ".weight");
    if (w.ne[0] != n_in || w.rows() != n_out) throw std::runtime_error(name + ": unexpected shape");
    matmul(m, w, w.data, n_out, x, T, n_in, y, n_out);
    if (const Tensor * b = m.find(name + ".bias")) {
        const float * bv = (const float *)b->data;
        for (size_t t = 0; t < T; ++t)
            for (size_t o = 0; o < n_out; ++o) y[t * n_out + o] += bv[o];
    }
    if (adapters && !m.loras.empty()) {
        for (size_t t = 0; t < T; ++t) apply_lora(m, adapters[t], name + ".weight", x + t * n_in, n_in, y + t * n_out, n_out);
    }
}

// One decode over a step plan, tokens batched in row-major order
// (crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:2572-2603).
void forward(Ctx & c, size_t n_rows, const int32_t * slot, const uint32_t * n, const int32_t * pos0, const uint8_t * sample,
             const int32_t * tokens, const int32_t * adapter, float * out_logits) {
    Model & m = *c.m;
    size_t T = 0;
    for (size_t r = 0; r < n_rows; ++r) T += n[r];
    std::vector<int32_t> tslot(T), tpos(T), tadapter(T);
    std::vector<size_t> out_tok;
    {
        size_t i = 0;
        for (size_t r = 0; r < n_rows; ++r) {
            for (uint32_t j = 0; j < n[r]; ++j, ++i) {
                tslot[i] = slot[r];
                tpos[i] = pos0[r] + (int32_t)j;
                tadapter[i] = adapter ? adapter[r] : 0;
            }
            if (sample[r]) out_tok.push_back(i - 1);
        }
    }
    const size_t d = m.d, hd = m.head_dim, dq = (size_t)m.n_head * hd, dkv = (size_t)m.n_head_kv * hd;
    std::vector<float> x(T * d), h(T * d), q(T * dq), k(T * dkv), v(T * dkv), att(T * dq), o(T * d);
    {
        const Tensor & e = m.need("token_embd.weight");
        const size_t rb = e.row_bytes();
        for (size_t t = 0; t < T; ++t) dequantize_row(e.type, e.data + (size_t)tokens[t] * rb, d, &x[t * d]);
    }
    // KV extents grow first so same-step rows of a slot see each other's cells.
    for (size_t t = 0; t < T; ++t) {
        SlotKV & s = c.slots[tslot[t]];
        if (s.k.empty()) { s.k.resize(m.n_layer); s.v.resize(m.n_layer); }
        if (s.pos_min < 0) s.pos_min = tpos[t];
        s.pos_min = std::min(s.pos_min, tpos[t]);
        s.pos_max = std::max(s.pos_max, tpos[t]);
        for (uint32_t l = 0; l < m.n_layer; ++l) {
            if (s.k[l].size() < (size_t)(s.pos_max + 1) * dkv) {
                s.k[l].resize((size_t)(s.pos_max + 1) * dkv);
                s.v[l].resize((size_t)(s.pos_max + 1) * dkv);
            }
        }
    }
    const bool moe = m.n_expert > 0;
    if (moe) c.last_routes.assign((size_t)m.n_layer * T * m.n_expert_used, -1);
    if (moe) c.last_route_margins.assign((size_t)m.n_layer * T, 0.f);
    const float att_scale = 1.0f / std::sqrt((float)hd);
    const uint32_t group = m.n_head / m.n_head_kv;
    for (uint32_t l = 0; l < m.n_layer; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        const float * wn = vec_f32(m, p + "attn_norm.weight");
        for (size_t t = 0; t < T; ++t) rms_norm(&x[t * d], wn, d, m.eps, &h[t * d]);
        linear(m, p + "attn_q", h.data(), T, d, q.data(), dq, tadapter.data());
        linear(m, p + "attn_k", h.data(), T, d, k.data(), dkv, tadapter.data());
        linear(m, p + "attn_v", h.data(), T, d, v.data(), dkv, tadapter.data());
        if (const Tensor * qn = m.find(p + "attn_q_norm.weight")) {
            const float * kn = vec_f32(m, p + "attn_k_norm.weight");
            std::vector<float> tmp(std::max(dq, dkv));
            for (size_t t = 0; t < T; ++t) {
                rms_norm(&q[t * dq], (const float *)qn->data, dq, m.eps, tmp.data());
                std::copy(tmp.begin(), tmp.begin() + dq, &q[t * dq]);
                rms_norm(&k[t * dkv], kn, dkv, m.eps, tmp.data());
                std::copy(tmp.begin(), tmp.begin() + dkv, &k[t * dkv]);
            }
        }
        for (size_t t = 0; t < T; ++t) {
            rope(&q[t * dq], m.n_head, hd, m.n_rot, m.neox, tpos[t], m.inv_freq);
            rope(&k[t * dkv], m.n_head_kv, hd, m.n_rot, m.neox, tpos[t], m.inv_freq);
            SlotKV & s = c.slots[tslot[t]];
            float * kd = &s.k[l][(size_t)tpos[t] * dkv];
            float * vd = &s.v[l][(size_t)tpos[t] * dkv];
            kv_store_row(c.kv_dtype, &k[t * dkv], kd, dkv);
            kv_store_row(c.kv_dtype, &v[t * dkv], vd, dkv);
        }
#pragma omp parallel for schedule(dynamic)
        for (int64_t th = 0; th < (int64_t)(T * m.n_head); ++th) {
            const size_t t = th / m.n_head, hq = th % m.n_head, hk = hq / group;
            const SlotKV & s = c.slots[tslot[t]];
            const int32_t p0 = s.pos_min, p1 = tpos[t];
            std::vector<float> sc(p1 - p0 + 1);
            const float * qv = &q[t * dq + hq * hd];
            float mx = -INFINITY;
            for (int32_t pp = p0; pp <= p1; ++pp) {
                const float * kv = &s.k[l][(size_t)pp * dkv + hk * hd];
                float acc = 0.f;
                for (size_t i = 0; i < hd; ++i) acc += qv[i] * kv[i];
                sc[pp - p0] = acc * att_scale;
                mx = std::max(mx, sc[pp - p0]);
            }
            float sum = 0.f;
            for (float & e : sc) { e = std::exp(e - mx); sum += e; }
            float * ov = &att[t * dq + hq * hd];
            for (size_t i = 0; i < hd; ++i) ov[i] = 0.f;
            for (int32_t pp = p0; pp <= p1; ++pp) {
                const float w = sc[pp - p0];
                const float * vv = &s.v[l][(size_t)pp * dkv + hk * hd];
                for (size_t i = 0; i < hd; ++i) ov[i] += w * vv[i];
            }
            const float inv = 1.0f / sum;
            for (size_t i = 0; i < hd; ++i) ov[i] *= inv;
        }
        linear(m, p + "attn_output", att.data(), T, dq, o.data(), d, tadapter.data());
        for (size_t i = 0; i < T * d; ++i) x[i] += o[i];
        const float * fn = vec_f32(m, p + "ffn_norm.weight");
        for (size_t t = 0; t < T; ++t) rms_norm(&x[t * d], fn, d, m.eps, &h[t * d]);
        if (!moe) {
            std::vector<float> gate(T * m.ff), up(T * m.ff);
            linear(m, p + "ffn_gate", h.data(), T, d, gate.data(), m.ff, tadapter.data());
            linear(m, p + "ffn_up", h.data(), T, d, up.data(), m.ff, tadapter.data());
            for (size_t i = 0; i < T * m.ff; ++i) {
                const float g = gate[i];
                gate[i] = g / (1.0f + std::exp(-g)) * up[i];
            }
            linear(m, p + "ffn_down", gate.data(), T, m.ff, o.data(), d, tadapter.data());
        } else {
            const Tensor & router = m.need(p + "ffn_gate_inp.weight");
            const Tensor & ge = m.need(p + "ffn_gate_exps.weight");
            const Tensor & ue = m.need(p + "ffn_up_exps.weight");
            const Tensor & de = m.need(p + "ffn_down_exps.weight");
            const size_t E = m.n_expert, K = m.n_expert_used, ff = m.ff;
            std::vector<float> logits(T * E);
            matmul(m, router, router.data, E, h.data(), T, d, logits.data(), E);
            std::vector<float> gate(ff), up(ff), y(d);
            for (size_t t = 0; t < T; ++t) {
                float * lg = &logits[t * E];
                float mx = -INFINITY;
                for (size_t e = 0; e < E; ++e) mx = std::max(mx, lg[e]);
                float sum = 0.f;
                std::vector<float> prob(E);
                for (size_t e = 0; e < E; ++e) { prob[e] = std::exp(lg[e] - mx); sum += prob[e]; }
                for (size_t e = 0; e < E; ++e) prob[e] /= sum;
                std::vector<int32_t> order(E);
                std::iota(order.begin(), order.end(), 0);
                std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return prob[a] > prob[b]; });
                std::vector<int32_t> sel(order.begin(), order.begin() + K);
                for (size_t j = 0; j < K; ++j) c.last_routes[((size_t)l * T + t) * K + j] = sel[j];
                float margin = INFINITY;
                for (size_t j = 0; j < K && j + 1 < E; ++j) margin = std::min(margin, prob[order[j]] - prob[order[j + 1]]);
                c.last_route_margins[(size_t)l * T + t] = margin;
                // accumulate in ascending expert id so the sum does not depend on how experts are placed
                std::sort(sel.begin(), sel.end());
                float * ot = &o[t * d];
                for (size_t i = 0; i < d; ++i) ot[i] = 0.f;
                for (int32_t e : sel) {
                    matmul(m, ge, ge.data + (size_t)e * ff * ge.row_bytes(), ff, &h[t * d], 1, d, gate.data(), ff);
                    matmul(m, ue, ue.data + (size_t)e * ff * ue.row_bytes(), ff, &h[t * d], 1, d, up.data(), ff);
                    for (size_t i = 0; i < ff; ++i) gate[i] = gate[i] / (1.0f + std::exp(-gate[i])) * up[i];
                    matmul(m, de, de.data + (size_t)e * d * de.row_bytes(), d, gate.data(), 1, ff, y.data(), d);
                    for (size_t i = 0; i < d; ++i) ot[i] += prob[e] * y[i];
                }
            }
        }
        for (size_t i = 0; i < T * d; ++i) x[i] += o[i];
    }
    if (!out_tok.empty() && out_logits) {
        const float * on = vec_f32(m, "output_norm.weight");
        const size_t S = out_tok.size();
        std::vector<float> hs(S * d);
        std::vector<int32_t> ads(S);
        for (size_t s = 0; s < S; ++s) {
            rms_norm(&x[out_tok[s] * d], on, d, m.eps, &hs[s * d]);
            ads[s] = tadapter[out_tok[s]];
        }
        const std::string head = m.find("output.weight") ? "output" : "token_embd";
        const Tensor & w = m.need(head + ".weight");
        matmul(m, w, w.data, m.vocab, hs.data(), S, d, out_logits, m.vocab);
        if (const Tensor * b = m.find("output.bias")) {
            const float * bv = (const float *)b->data;
            for (size_t s = 0; s < S; ++s)
                for (size_t i = 0; i < m.vocab; ++i) out_logits[s * m.vocab + i] += bv[i];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Sampling oracle (crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:41-51,103-225,718-875,2942-2985)

struct Scratch {
    float max = 0.f;
    double total = 0.0;
    std::vector<double> probs;
    std::vector<int32_t> order;
    std::vector<float> t;
};

void log_softmax_terms(const float * logits, size_t n, float & mx, double & log_sum) {
    mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) mx = std::max(mx, logits[i]);
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += std::exp((double)logits[i] - mx);
    log_sum = std::log(sum);
}

int32_t draw_from_probs(std::vector<double> & probs, size_t n, float top_p, std::mt19937 & rng, Scratch & sc, double & denom, bool truncate) {
    const double total = sc.total;
    if (top_p == 1.0f) {
        std::uniform_real_distribution<double> uniform(0.0, total);
        const double draw = uniform(rng);
        double acc = 0.0;
        for (size_t i = 0; i < n; ++i) {
            acc += probs[i];
            if (probs[i] > 0.0 && draw <= acc) { denom = total; return (int32_t)i; }
        }
        denom = total;
        return (int32_t)(n - 1);
    }
    std::vector<int32_t> & order = sc.order;
    order.resize(n);
    std::iota(order.begin(), order.end(), 0);
    const double target = (double)top_p * total;
    double kept = 0.0;
    size_t n_keep = 0;
    std::sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return probs[a] > probs[b]; });
    while (n_keep < n) {
        kept += probs[order[n_keep]];
        ++n_keep;
        if (kept >= target) break;
    }
    if (truncate) {
        for (size_t i = n_keep; i < n; ++i) probs[order[i]] = 0.0;
    }
    std::uniform_real_distribution<double> uniform(0.0, kept);
    const double draw = uniform(rng);
    double acc = 0.0;
    for (size_t i = 0; i < n_keep; ++i) {
        acc += probs[order[i]];
        if (draw <= acc) { denom = kept; return order[i]; }
    }
    denom = kept;
    return order[n_keep - 1];
}

int32_t sample_token(const float * logits, size_t n, float temperature, float top_p, std::mt19937 & rng, Scratch & sc) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) mx = std::max(mx, logits[i]);
    if (!std::isfinite(mx)) return -1;
    sc.max = mx;
    sc.probs.resize(n);
    double total = 0.0;
    for (size_t i = 0; i < n; ++i) {
        sc.probs[i] = std::exp(((double)logits[i] - mx) / temperature);
        total += sc.probs[i];
    }
    sc.total = total;
    double denom = 0.0;
    return draw_from_probs(sc.probs, n, top_p, rng, sc, denom, false);
}

void top_token_logprobs(const float * logits, size_t n, size_t k, int32_t * ids, float * lps) {
    float mx;
    double ls;
    log_softmax_terms(logits, n, mx, ls);
    std::vector<int32_t> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](int32_t a, int32_t b) {
        if (logits[a] != logits[b]) return logits[a] > logits[b];
        return a < b;
    });
    for (size_t j = 0; j < k; ++j) {
        ids[j] = order[j];
        lps[j] = (float)((double)logits[order[j]] - mx - ls);
    }
}

struct V2Params {
    float temperature, top_p;
    int32_t top_k;
    float min_p, repeat_penalty, frequency_penalty, presence_penalty;
    uint32_t penalty_window, n_logit_bias;
    const int32_t * bias_ids;
    const float * bias_values;
};

int32_t sample_token_v2(const float * logits, size_t n, const V2Params & p, std::mt19937 & rng, Scratch & sc, const int32_t * history,
                        size_t n_history, float * out_sampled_logprob, int32_t * top_ids, float * top_lps, size_t k) {
    std::vector<float> & t = sc.t;
    t.assign(logits, logits + n);
    for (uint32_t i = 0; i < p.n_logit_bias; ++i) t[p.bias_ids[i]] += p.bias_values[i];
    const bool any_penalty = p.repeat_penalty != 1.0f || p.frequency_penalty != 0.0f || p.presence_penalty != 0.0f;
    if (any_penalty && n_history > 0) {
        const size_t window = p.penalty_window == 0 ? n_history : std::min<size_t>(p.penalty_window, n_history);
        std::unordered_map<int32_t, int32_t> counts;
        for (size_t i = n_history - window; i < n_history; ++i) counts[history[i]]++;
        for (const auto & e : counts) {
            const int32_t id = e.first, count = e.second;
            if (t[id] <= 0.0f) t[id] *= p.repeat_penalty; else t[id] /= p.repeat_penalty;
            t[id] -= (float)count * p.frequency_penalty + (float)(count > 0) * p.presence_penalty;
        }
    }
    if (p.top_k > 0 && (size_t)p.top_k < n) {
        std::vector<int32_t> & order = sc.order;
        order.resize(n);
        std::iota(order.begin(), order.end(), 0);
        const size_t keep = (size_t)p.top_k;
        std::partial_sort(order.begin(), order.begin() + keep, order.end(), [&](int32_t a, int32_t b) { return t[a] > t[b]; });
        for (size_t i = keep; i < n; ++i) t[order[i]] = -INFINITY;
    }
    if (p.min_p > 0.0f) {
        float ml = -INFINITY;
        for (size_t i = 0; i < n; ++i) ml = std::max(ml, t[i]);
        const float thr = ml + std::log(p.min_p);
        for (size_t i = 0; i < n; ++i) if (t[i] < thr) t[i] = -INFINITY;
    }
    float mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) mx = std::max(mx, t[i]);
    sc.max = mx;
    sc.probs.resize(n);
    double total = 0.0;
    for (size_t i = 0; i < n; ++i) {
        sc.probs[i] = std::exp(((double)t[i] - mx) / p.temperature);
        total += sc.probs[i];
    }
    sc.total = total;
    double denom = 0.0;
    const int32_t token = draw_from_probs(sc.probs, n, p.top_p, rng, sc, denom, true);
    sc.total = denom;
    if (k > 0 && top_ids && top_lps) {
        std::vector<int32_t> & order = sc.order;
        order.resize(n);
        std::iota(order.begin(), order.end(), 0);
        std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](int32_t a, int32_t b) {
            if (sc.probs[a] != sc.probs[b]) return sc.probs[a] > sc.probs[b];
            return a < b;
        });
        for (size_t j = 0; j < k; ++j) {
            top_ids[j] = order[j];
            top_lps[j] = (float)std::log(sc.probs[order[j]] / denom);
        }
    }
    if (out_sampled_logprob) *out_sampled_logprob = (float)std::log(sc.probs[token] / denom);
    return token;
}

// ---------------------------------------------------------------------------------------------
// Restatement of this backend's own counter-based draw (not a reference function: the reference
// draws from std::mt19937, which a GPU cannot reproduce without serialising; the contract for
// seeded rows is "same distribution, reproducible for a fixed seed").
// Philox4x32-10 keyed by (seed, 0x5EEDB200), counter (draw index, 0, 0, 0); u in [0,1) from 53 bits.

void philox4x32(uint32_t key0, uint32_t key1, uint32_t c[4]) {
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ key0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ key1;
        const uint32_t n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        key0 += 0x9E3779B9u;
        key1 += 0xBB67AE85u;
    }
}

double philox_uniform(uint32_t seed, uint64_t draw) {
    uint32_t c[4] = {(uint32_t)draw, (uint32_t)(draw >> 32), 0, 0};
    philox4x32(seed, 0x5EEDB200u, c);
    const uint64_t bits = (((uint64_t)c[0] << 32) | c[1]) >> 11;
    return (double)bits * (1.0 / 9007199254740992.0);
}

} // namespace

// =============================================================================================
// C API

extern "C" {

// Sets (n > 0) and reports the number of OpenMP threads the forward pass uses. A launcher may export
// OMP_NUM_THREADS=1 to its children; a timed baseline states its thread count instead of inheriting one.
int ora_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
}

const char * ora_last_error(void) { return g_error.c_str(); }

int ora_dequantize_row(uint32_t type, const uint8_t * src, size_t n, float * out) {
    return dequantize_row(type, src, n, out) ? 0 : -1;
}

float ora_half_to_f32(uint16_t h) { return half_to_f32(h); }
float ora_round_to_half(float v) { return round_to_half(v); }
float ora_e8m0_half(uint8_t x) { return e8m0_to_f32_half(x); }

// dst[row] = sum_col deq(a)[row][col] * b[col], serial f32
// The act = q8 form of the GEMV below: b re-quantised to the 8-bit block format of `type`'s dot product (F16: to f16)
int ora_mul_mat_vec_act_q8(uint32_t type, size_t n_row, size_t n_col, const uint8_t * a, const float * b, float * dst) {
    size_t be, bb;
    if (!geom(type, be, bb) || n_col % be || !act_q8_applies(type, n_col)) return -1;
    Tensor w;
    w.type = type;
    w.ne = {n_col, n_row};
    w.data = a;
    matmul_act_q8(w, a, n_row, b, 1, n_col, dst, n_row);
    return 0;
}

int ora_mul_mat_vec(uint32_t type, size_t n_row, size_t n_col, const uint8_t * a, const float * b, float * dst) {
    size_t be, bb;
    if (!geom(type, be, bb) || n_col % be) return -1;
    std::vector<float> row(n_col);
    for (size_t r = 0; r < n_row; ++r) {
        dequantize_row(type, a + r * (n_col / be * bb), n_col, row.data());
        float acc = 0.f;
        for (size_t c = 0; c < n_col; ++c) acc += row[c] * b[c];
        dst[r] = acc;
    }
    return 0;
}

void ora_rms_norm(const float * x, const float * w, size_t n, float eps, float * y) { rms_norm(x, w, n, eps, y); }

void * ora_model_load(const char * path) {
    try {
        auto m = std::make_unique<Model>();
        m->g = gguf_open(path);
        Gguf & g = *m->g;
        m->arch = g.str["general.architecture"];
        const std::string a = m->arch;
        if (a != "llama" && a != "qwen2" && a != "olmoe") throw std::runtime_error("unsupported architecture " + a);
        m->neox = a != "llama";
        m->n_layer = g.u32[a + ".block_count"];
        m->d = g.u32[a + ".embedding_length"];
        m->n_head = g.u32[a + ".attention.head_count"];
        m->n_head_kv = g.u32.count(a + ".attention.head_count_kv") ? g.u32[a + ".attention.head_count_kv"] : m->n_head;
        m->head_dim = g.u32.count(a + ".attention.key_length") ? g.u32[a + ".attention.key_length"] : m->d / m->n_head;
        m->ff = g.u32[a + ".feed_forward_length"];
        m->eps = g.f32.count(a + ".attention.layer_norm_rms_epsilon") ? g.f32[a + ".attention.layer_norm_rms_epsilon"] : 1e-5f;
        m->rope_base = g.f32.count(a + ".rope.freq_base") ? g.f32[a + ".rope.freq_base"] : 10000.f;
        m->n_rot = g.u32.count(a + ".rope.dimension_count") ? g.u32[a + ".rope.dimension_count"] : m->head_dim;
        m->n_expert = g.u32.count(a + ".expert_count") ? g.u32[a + ".expert_count"] : 0;
        m->n_expert_used = g.u32.count(a + ".expert_used_count") ? g.u32[a + ".expert_used_count"] : 0;
        m->vocab = (uint32_t)m->need("token_embd.weight").ne[1];
        m->inv_freq.resize(m->n_rot / 2);
        for (uint32_t i = 0; i < m->n_rot / 2; ++i) m->inv_freq[i] = (float)std::pow((double)m->rope_base, -2.0 * i / m->n_rot);
        return m.release();
    } catch (const std::exception & e) {
        g_error = e.what();
        return nullptr;
    }
}

void ora_model_free(void * m) { delete (Model *)m; }

void ora_model_set_fast(void * m, int fast) { ((Model *)m)->fast = fast != 0; }

// act = q8 (1) or act = f32 (0, the default): see Model::act_q8
void ora_model_set_act_q8(void * m, int on) { ((Model *)m)->act_q8 = on != 0; }

// out: n_layer, d, n_head, n_head_kv, head_dim, ff, vocab, n_expert, n_expert_used, neox
void ora_model_info(void * mp, uint32_t * out) {
    Model & m = *(Model *)mp;
    const uint32_t v[10] = {m.n_layer, m.d, m.n_head, m.n_head_kv, m.head_dim, m.ff, m.vocab, m.n_expert, m.n_expert_used, m.neox};
    std::memcpy(out, v, sizeof v);
}

// Loads a LoRA adapter GGUF (general.type=adapter, adapter.lora.alpha; tensors
// `<weight>.lora_a` [in, r] and `<weight>.lora_b` [r, out];
// crates/retrograd-ffi/runtime/src/retro_lora.cpp:1019-1027,1144-1157). Returns its id (> 0).
int32_t ora_lora_load(void * mp, const char * path, float scale) {
    try {
        Model & m = *(Model *)mp;
        auto g = gguf_open(path);
        Lora lora;
        const float alpha = g->f32.count("adapter.lora.alpha") ? g->f32["adapter.lora.alpha"] : 0.f;
        for (auto & kv : g->tensors) {
            const std::string & name = kv.first;
            const std::string suffix = ".lora_a";
            if (name.size() <= suffix.size() || name.compare(name.size() - suffix.size(), suffix.size(), suffix) != 0) continue;
            const std::string target = name.substr(0, name.size() - suffix.size());
            const Tensor & A = kv.second;
            auto itb = g->tensors.find(target + ".lora_b");
            if (itb == g->tensors.end()) throw std::runtime_error("adapter lacks " + target + ".lora_b");
            const Tensor & B = itb->second;
            const uint32_t r = (uint32_t)A.ne[1];
            if (lora.rank && lora.rank != r) throw std::runtime_error("oracle supports one rank per adapter");
            lora.rank = r;
            std::vector<float> a(A.ne[0] * A.ne[1]), b(B.ne[0] * B.ne[1]);
            for (size_t j = 0; j < A.ne[1]; ++j) dequantize_row(A.type, A.data + j * A.row_bytes(), A.ne[0], &a[j * A.ne[0]]);
            for (size_t j = 0; j < B.ne[1]; ++j) dequantize_row(B.type, B.data + j * B.row_bytes(), B.ne[0], &b[j * B.ne[0]]);
            lora.ab[target] = {std::move(a), std::move(b)};
        }
        if (lora.rank == 0) throw std::runtime_error("adapter holds no lora tensors");
        lora.scale = (alpha != 0.f ? alpha / (float)lora.rank : 1.0f) * scale;
        const int32_t id = m.next_lora++;
        m.loras[id] = std::move(lora);
        return id;
    } catch (const std::exception & e) {
        g_error = e.what();
        return -1;
    }
}

// What a cache of `kv_dtype` returns for the row `src` of n values (n a multiple of 32 for the quantised types)
void ora_kv_round(int kv_dtype, const float * src, float * dst, uint64_t n) { kv_store_row(kv_dtype, src, dst, (size_t)n); }

// kv_dtype: retro_engine_kv_dtype (0 F32, 1 F16, 2 Q8_0, 3 Q4_0); the quantised types need head_dim % 32 == 0
void * ora_ctx_new(void * m, uint32_t n_slots, uint32_t n_ctx_seq, int kv_dtype) {
    Ctx * c = new Ctx{(Model *)m, n_slots, n_ctx_seq, kv_dtype, {}, {}};
    c->slots.resize(n_slots);
    return c;
}

void ora_ctx_free(void * c) { delete (Ctx *)c; }

// Batch maps of a step plan in the reference's order: row-major over rows, tokens in row order;
// the last token of a sampling row is its output (retro_gen_core.cpp:2579-2603).
// Outputs: tok_slot[T], tok_pos[T], tok_row[T], out_index[S], cu[n_rows+1]. Returns T; *n_out = S.
size_t ora_pack(size_t n_rows, const int32_t * slot, const uint32_t * n, const int32_t * pos0, const uint8_t * sample,
                int32_t * tok_slot, int32_t * tok_pos, int32_t * tok_row, int32_t * out_index, int32_t * cu, size_t * n_out) {
    size_t i = 0, s = 0;
    for (size_t r = 0; r < n_rows; ++r) {
        cu[r] = (int32_t)i;
        for (uint32_t j = 0; j < n[r]; ++j, ++i) {
            tok_slot[i] = slot[r];
            tok_pos[i] = pos0[r] + (int32_t)j;
            tok_row[i] = (int32_t)r;
        }
        if (sample[r]) out_index[s++] = (int32_t)(i - 1);
    }
    cu[n_rows] = (int32_t)i;
    *n_out = s;
    return i;
}

// Decodes the rows; writes logits of sampling rows (in row order) to out_logits [S, vocab].
int ora_step(void * cp, size_t n_rows, const int32_t * slot, const uint32_t * n, const int32_t * pos0, const uint8_t * sample,
             const int32_t * tokens, const int32_t * adapter, float * out_logits) {
    try {
        Ctx & c = *(Ctx *)cp;
        for (size_t r = 0; r < n_rows; ++r) {
            if (slot[r] < 0 || (uint32_t)slot[r] >= c.n_slots) throw std::runtime_error("slot out of range");
            if (pos0[r] < 0 || (uint64_t)pos0[r] + n[r] > c.n_ctx_seq) throw std::runtime_error("positions exceed the context");
        }
        forward(c, n_rows, slot, n, pos0, sample, tokens, adapter, out_logits);
        return 0;
    } catch (const std::exception & e) {
        g_error = e.what();
        return -1;
    }
}

// Expert ids the last step selected: [layer][token][k], selection order.
size_t ora_last_route_margins(void * cp, float * out, size_t n_max) {
    Ctx & c = *(Ctx *)cp;
    const size_t n = std::min(n_max, c.last_route_margins.size());
    if (out) std::memcpy(out, c.last_route_margins.data(), n * 4);
    return c.last_route_margins.size();
}

size_t ora_last_routes(void * cp, int32_t * out, size_t n_max) {
    Ctx & c = *(Ctx *)cp;
    const size_t n = std::min(n_max, c.last_routes.size());
    if (out) std::memcpy(out, c.last_routes.data(), n * 4);
    return c.last_routes.size();
}

int ora_seq_pos(void * cp, int32_t slot, int32_t * pmin, int32_t * pmax) {
    Ctx & c = *(Ctx *)cp;
    *pmin = c.slots[slot].pos_min;
    *pmax = c.slots[slot].pos_min < 0 ? -1 : c.slots[slot].pos_max;
    return 0;
}

// [p0, p1), negative = open (retro_lora_train.h:2721-2729). Only whole or tail removals.
int ora_seq_rm(void * cp, int32_t slot, int32_t p0, int32_t p1) {
    Ctx & c = *(Ctx *)cp;
    SlotKV & s = c.slots[slot];
    if (s.pos_min < 0) return 0;
    if (p0 < 0) p0 = 0;
    if (p1 < 0) p1 = s.pos_max + 1;
    if (p0 <= s.pos_min && p1 > s.pos_max) { s = SlotKV{}; return 0; }
    if (p1 > s.pos_max && p0 > s.pos_min) { s.pos_max = p0 - 1; return 0; }
    if (p0 > s.pos_max || p1 <= s.pos_min) return 0;
    return -1;
}

int ora_seq_cp(void * cp, int32_t src, int32_t dst, int32_t p0, int32_t p1) {
    Ctx & c = *(Ctx *)cp;
    if (src == dst) return 0;
    SlotKV & s = c.slots[src];
    SlotKV & t = c.slots[dst];
    if (s.pos_min < 0) return 0;
    if (p0 < 0) p0 = 0;
    if (p1 < 0) p1 = s.pos_max + 1;
    p0 = std::max(p0, s.pos_min);
    p1 = std::min(p1, s.pos_max + 1);
    if (p0 >= p1) return 0;
    const size_t dkv = (size_t)c.m->n_head_kv * c.m->head_dim;
    if (t.k.empty()) { t.k.resize(c.m->n_layer); t.v.resize(c.m->n_layer); }
    for (uint32_t l = 0; l < c.m->n_layer; ++l) {
        if (t.k[l].size() < (size_t)p1 * dkv) { t.k[l].resize((size_t)p1 * dkv); t.v[l].resize((size_t)p1 * dkv); }
        std::copy(s.k[l].begin() + (size_t)p0 * dkv, s.k[l].begin() + (size_t)p1 * dkv, t.k[l].begin() + (size_t)p0 * dkv);
        std::copy(s.v[l].begin() + (size_t)p0 * dkv, s.v[l].begin() + (size_t)p1 * dkv, t.v[l].begin() + (size_t)p0 * dkv);
    }
    if (t.pos_min < 0) {
        t.pos_min = p0;
        t.pos_max = p1 - 1;
    } else {
        t.pos_min = std::min(t.pos_min, p0);
        t.pos_max = std::max(t.pos_max, p1 - 1);
    }
    return 0;
}

void * ora_rng_new(uint32_t seed) { return new std::mt19937(seed); }
void ora_rng_free(void * r) { delete (std::mt19937 *)r; }

void ora_log_softmax_terms(const float * logits, size_t n, float * mx, double * log_sum) { log_softmax_terms(logits, n, *mx, *log_sum); }

// v1 row of the step: token, plus the logprob expression the step reports
// (retro_gen_core.cpp:2753-2765).
int32_t ora_sample_token(const float * logits, size_t n, float temperature, float top_p, void * rng, float * out_logprob) {
    Scratch sc;
    const int32_t token = sample_token(logits, n, temperature, top_p, *(std::mt19937 *)rng, sc);
    if (token >= 0 && out_logprob) {
        if (temperature == 1.0f) {
            *out_logprob = (float)((double)logits[token] - sc.max - std::log(sc.total));
        } else {
            float mx;
            double ls;
            log_softmax_terms(logits, n, mx, ls);
            *out_logprob = (float)((double)logits[token] - mx - ls);
        }
    }
    return token;
}

void ora_top_token_logprobs(const float * logits, size_t n, size_t k, int32_t * ids, float * lps) { top_token_logprobs(logits, n, k, ids, lps); }

int32_t ora_sample_token_v2(const float * logits, size_t n, float temperature, float top_p, int32_t top_k, float min_p,
                            float repeat_penalty, float frequency_penalty, float presence_penalty, uint32_t penalty_window,
                            uint32_t n_logit_bias, const int32_t * bias_ids, const float * bias_values, void * rng,
                            const int32_t * history, size_t n_history, float * out_logprob, float * out_sampled_logprob,
                            int32_t * top_ids, float * top_lps, size_t k) {
    Scratch sc;
    const V2Params p{temperature, top_p, top_k, min_p, repeat_penalty, frequency_penalty, presence_penalty,
                     penalty_window, n_logit_bias, bias_ids, bias_values};
    const int32_t token = sample_token_v2(logits, n, p, *(std::mt19937 *)rng, sc, history, n_history, out_sampled_logprob, top_ids, top_lps, k);
    if (token >= 0 && out_logprob) {
        float mx;
        double ls;
        log_softmax_terms(logits, n, mx, ls);
        *out_logprob = (float)((double)logits[token] - mx - ls);
    }
    return token;
}

double ora_philox_uniform(uint32_t seed, uint64_t draw) { return philox_uniform(seed, draw); }

// This backend's seeded draw, restated on the CPU: probabilities as the reference forms them
// (exp((l - max)/T) in double), nucleus = the highest-probability tokens (ties by ascending id)
// whose mass first reaches top_p * total, and a cumulative draw over the kept tokens in id order.
// Writes the boundary distance of the draw to *out_margin (relative to the kept mass) so a
// comparison can recognise a draw that sits on a rounding boundary.
int32_t ora_sample_philox(const float * logits, size_t n, float temperature, float top_p, uint32_t seed, uint64_t draw_index,
                          double * out_margin) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) mx = std::max(mx, logits[i]);
    std::vector<double> probs(n);
    double total = 0.0;
    for (size_t i = 0; i < n; ++i) { probs[i] = std::exp(((double)logits[i] - mx) / temperature); total += probs[i]; }
    std::vector<uint8_t> keep(n, 1);
    double kept = total;
    if (top_p < 1.0f) {
        std::vector<int32_t> order(n);
        std::iota(order.begin(), order.end(), 0);
        std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return probs[a] > probs[b]; });
        std::fill(keep.begin(), keep.end(), 0);
        const double target = (double)top_p * total;
        kept = 0.0;
        for (size_t i = 0; i < n; ++i) {
            keep[order[i]] = 1;
            kept += probs[order[i]];
            if (kept >= target) break;
        }
        kept = 0.0;
        for (size_t i = 0; i < n; ++i) if (keep[i]) kept += probs[i];
    }
    const double draw = philox_uniform(seed, draw_index) * kept;
    double acc = 0.0;
    int32_t last = -1;
    double margin = 1.0;
    int32_t pick = -1;
    for (size_t i = 0; i < n; ++i) {
        if (!keep[i] || probs[i] <= 0.0) continue;
        last = (int32_t)i;
        acc += probs[i];
        margin = std::min(margin, std::fabs(draw - acc) / kept);
        if (pick < 0 && draw < acc) pick = (int32_t)i;
    }
    if (out_margin) *out_margin = margin;
    return pick >= 0 ? pick : last;
}

} // extern "C"
