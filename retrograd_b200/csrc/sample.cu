// On-device sampling for the step's output rows: one 1024-thread block per logits row.
//
// What is reproduced from the reference's CPU oracle
// (crates/retrograd-ffi/runtime/src/retro_gen_core.cpp:41-51,103-225,718-875,2942-2985):
//   - logprob = logit - max - log(sum exp(logit - max)), the sum taken in double;
//   - top logprobs ordered by (logit desc, id asc);
//   - probabilities p_i = exp((l_i - max) / T) in double; nucleus = highest-probability tokens
//     whose mass first reaches top_p * total; v2 order bias -> penalties -> top_k -> min_p ->
//     temperature -> top_p -> draw.
// What differs by design: the uniform draw comes from a counter-based generator (Philox4x32-10
// keyed by the request seed, counter = the request's draw index) instead of std::mt19937, and
// the cumulative draw walks the kept tokens in id order. Greedy rows (top_k == 1, or a nucleus
// that holds a single token) pick the arg-max with the lowest id on ties and are exact.
// Every reduction has a fixed order, so a (seed, draw index, logits) triple always yields the
// same token.

#include "kernels.cuh"

#include <cfloat>

namespace rb200 {

namespace {

constexpr int kThreads = 1024;
constexpr uint32_t kFlagV2 = 1u, kFlagWantLogprob = 2u, kFlagGreedyFast = 4u;

struct Shared {
    double dwarp[32];
    float fwarp[32];
    int32_t iwarp[32];
    unsigned long long hist[256];
    double dval;
    float fval;
    int32_t ival;
    int32_t ival2;
    uint32_t uval;
    unsigned long long ullval;
    unsigned long long ullval2;
};

__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ void philox4x32(uint32_t k0, uint32_t k1, uint32_t (&c)[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

__device__ double philox_uniform(uint32_t seed, uint32_t draw_lo, uint32_t draw_hi) {
    uint32_t c[4] = {draw_lo, draw_hi, 0u, 0u};
    philox4x32(seed, 0x5EEDB200u, c);
    const uint64_t bits = (((uint64_t)c[0] << 32) | c[1]) >> 11;
    return (double)bits * (1.0 / 9007199254740992.0);
}

// (value desc, id asc) arg-max over the block. Result broadcast to every thread.
__device__ void block_argmax(Shared & sh, float v, int32_t id, float & out_v, int32_t & out_id) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int32_t oi = __shfl_xor_sync(0xffffffffu, id, o);
        if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; }
    }
    __syncthreads();
    if (lane == 0) { sh.fwarp[wid] = v; sh.iwarp[wid] = id; }
    __syncthreads();
    if (wid == 0) {
        v = sh.fwarp[lane];
        id = sh.iwarp[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int32_t oi = __shfl_xor_sync(0xffffffffu, id, o);
            if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; }
        }
        if (lane == 0) { sh.fval = v; sh.ival = id; }
    }
    __syncthreads();
    out_v = sh.fval;
    out_id = sh.ival;
}

// Fixed-order sum of doubles over the block, broadcast.
__device__ double block_sum(Shared & sh, double v) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh.dwarp[wid] = v;
    __syncthreads();
    if (wid == 0) {
        v = sh.dwarp[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) sh.dval = v;
    }
    __syncthreads();
    return sh.dval;
}

// Exclusive prefix over threads in thread order; *total receives the block sum.
__device__ double block_exclusive_scan(Shared & sh, double v, double * total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    double inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double u = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += u;
    }
    __syncthreads();
    if (lane == 31) sh.dwarp[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        double w = sh.dwarp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double u = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += u;
        }
        sh.dwarp[lane] = w;
    }
    __syncthreads();
    const double pre = (wid ? sh.dwarp[wid - 1] : 0.0) + inc - v;
    if (total) *total = sh.dwarp[31];
    return pre;
}

__device__ int32_t block_exclusive_scan_int(Shared & sh, int32_t v, int32_t * total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int32_t u = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += u;
    }
    __syncthreads();
    if (lane == 31) sh.iwarp[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int32_t w = sh.iwarp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t u = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += u;
        }
        sh.iwarp[lane] = w;
    }
    __syncthreads();
    const int32_t pre = (wid ? sh.iwarp[wid - 1] : 0) + inc - v;
    if (total) *total = sh.iwarp[31];
    return pre;
}

// Radix select over the descending order of logits. `by_mass`: weights are fixed-point
// probabilities and the walk stops when the accumulated weight reaches `target`; otherwise
// weights are 1 (a count). Returns the key of the last kept value in *thr_key, and the weight
// accumulated by strictly greater keys in *above.
__device__ void radix_select(Shared & sh, const float * __restrict__ l, int V, bool by_mass, float tmax, double inv_t,
                             unsigned long long target, uint32_t * thr_key, unsigned long long * above) {
    uint32_t prefix = 0;
    unsigned long long acc_above = 0;
    for (int digit = 3; digit >= 0; --digit) {
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.hist[b] = 0ull;
        __syncthreads();
        const int shift = digit * 8;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = l[i];
            const uint32_t key = order_key(v);
            if (digit == 3 || (key >> (shift + 8)) == prefix) {
                unsigned long long w = 1ull;
                if (by_mass) w = (unsigned long long)(exp(((double)v - (double)tmax) * inv_t) * 1099511627776.0);
                if (w) atomicAdd(&sh.hist[(key >> shift) & 255u], w);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long acc = acc_above;
            int pick = 0;
            for (int b = 255; b >= 0; --b) {
                if (acc + sh.hist[b] >= target) { pick = b; break; }
                acc += sh.hist[b];
            }
            sh.ullval = acc;
            sh.uval = (prefix << 8) | (uint32_t)pick;
        }
        __syncthreads();
        prefix = sh.uval;
        acc_above = sh.ullval;
    }
    *thr_key = prefix;
    *above = acc_above;
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const float * __restrict__ raw_logits, float * __restrict__ work_logits, int V,
                                                          const SampleDesc * __restrict__ descs, const LogitEdit * __restrict__ edits,
                                                          const uint32_t * __restrict__ masks, SampleOut * __restrict__ outs,
                                                          int32_t * __restrict__ top_ids, float * __restrict__ top_lps, int top_stride) {
    __shared__ Shared sh;
    const int row = blockIdx.x;
    const SampleDesc d = descs[row];
    if (d.flags & kFlagGreedyFast) return;      // served by the chunked arg-max kernels below
    const bool v2 = (d.flags & kFlagV2) != 0;
    // v2 rows transform a private copy of their row; v1 rows only read the raw one
    const float * raw = raw_logits + (size_t)row * V;
    float * l = v2 ? work_logits + (size_t)row * V : const_cast<float *>(raw);
    const int tid = threadIdx.x;

    // ---- temperature-1 statistics of the raw row
    float rmax = -INFINITY;
    int32_t rarg = 0x7fffffff;
    for (int i = tid; i < V; i += kThreads) {
        const float v = l[i];
        if (v > rmax) { rmax = v; rarg = i; }
    }
    block_argmax(sh, rmax, rarg, rmax, rarg);
    double part = 0.0;
    for (int i = tid; i < V; i += kThreads) part += exp((double)l[i] - (double)rmax);
    const double rlog = log(block_sum(sh, part));

    // ---- raw top logprobs (v1 rows report the temperature-1 policy)
    const uint32_t n_top = min(d.n_top, (uint32_t)min(top_stride, V));
    if (!v2 && n_top > 0) {
        float pv = INFINITY;
        int32_t pid = -1;
        for (uint32_t j = 0; j < n_top; ++j) {
            float bv = -INFINITY;
            int32_t bi = 0x7fffffff;
            for (int i = tid; i < V; i += kThreads) {
                const float v = l[i];
                const bool after = v < pv || (v == pv && i > pid);
                if (after && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
            }
            block_argmax(sh, bv, bi, bv, bi);
            if (tid == 0) {
                top_ids[(size_t)row * top_stride + j] = bi;
                top_lps[(size_t)row * top_stride + j] = (float)((double)bv - (double)rmax - rlog);
            }
            pv = bv;
            pid = bi;
        }
    }

    // ---- v2 transformations, on the row's working copy
    const uint32_t n_edits = d.edit_end - d.edit_begin;
    __syncthreads();
    if (v2) {
        // logit_bias and penalties: one merged edit per distinct id
        for (uint32_t e = tid; e < n_edits; e += kThreads) {
            const LogitEdit ed = edits[d.edit_begin + e];
            float t = l[ed.id] + ed.bias;
            if (ed.repeat != 1.0f) t = t <= 0.0f ? t * ed.repeat : t / ed.repeat;
            t -= ed.subtract;
            l[ed.id] = t;
        }
        __syncthreads();
        // grammar mask: one bit per token, tokens the grammar cannot continue with drop out here
        if (d.pad[0] != 0 && masks) {
            const uint32_t * bits = masks + (d.pad[0] - 1);
            for (int i = tid; i < V; i += kThreads)
                if (!((bits[i >> 5] >> (i & 31)) & 1u)) l[i] = -INFINITY;
            __syncthreads();
        }
        // top_k (count based, ties keep the lowest ids)
        if (d.top_k > 0 && d.top_k < V) {
            uint32_t thr;
            unsigned long long above;
            radix_select(sh, l, V, false, 0.f, 0.0, (unsigned long long)d.top_k, &thr, &above);
            const int32_t ties_keep = d.top_k - (int32_t)above;
            const int chunk = (V + kThreads - 1) / kThreads;
            const int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);
            int32_t my_ties = 0;
            for (int i = c0; i < c1; ++i) my_ties += order_key(l[i]) == thr;
            int32_t rank = block_exclusive_scan_int(sh, my_ties, nullptr);
            for (int i = c0; i < c1; ++i) {
                const uint32_t key = order_key(l[i]);
                if (key < thr) {
                    l[i] = -INFINITY;
                } else if (key == thr) {
                    if (rank >= ties_keep) l[i] = -INFINITY;
                    ++rank;
                }
            }
            __syncthreads();
        }
        if (d.min_p > 0.0f) {
            float mv = -INFINITY;
            int32_t mi = 0;
            for (int i = tid; i < V; i += kThreads) mv = fmaxf(mv, l[i]);
            block_argmax(sh, mv, 0, mv, mi);
            const float thr = mv + logf(d.min_p);
            for (int i = tid; i < V; i += kThreads) if (l[i] < thr) l[i] = -INFINITY;
            __syncthreads();
        }
    }

    // ---- sampling distribution
    float tmax = rmax;
    int32_t targ = rarg;
    if (v2) {
        tmax = -INFINITY;
        targ = 0x7fffffff;
        for (int i = tid; i < V; i += kThreads) {
            const float v = l[i];
            if (v > tmax) { tmax = v; targ = i; }
        }
        block_argmax(sh, tmax, targ, tmax, targ);
    }
    const double inv_t = 1.0 / (double)d.temperature;
    part = 0.0;
    for (int i = tid; i < V; i += kThreads) part += exp(((double)l[i] - (double)tmax) * inv_t);
    const double total = block_sum(sh, part);

    int32_t token;
    double kept = total;
    uint32_t thr = 0;
    int32_t ties_keep = 0x7fffffff;
    const bool single = (v2 && d.top_k == 1) || (double)d.top_p * total <= 1.0;
    const bool nucleus = !single && d.top_p < 1.0f;
    if (nucleus) {
        // fixed-point masses make the selection independent of the order atomics land in
        double fp = 0.0;
        for (int i = tid; i < V; i += kThreads)
            fp += (double)(unsigned long long)(exp(((double)l[i] - (double)tmax) * inv_t) * 1099511627776.0);
        const double total_fixed = block_sum(sh, fp);
        unsigned long long target = (unsigned long long)((double)d.top_p * total_fixed);
        if (target < 1ull) target = 1ull;
        unsigned long long above;
        radix_select(sh, l, V, true, tmax, inv_t, target, &thr, &above);
        // weight of one token at the threshold
        float thr_val;
        {
            const uint32_t u = (thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr;
            thr_val = __uint_as_float(u);
        }
        const unsigned long long w = (unsigned long long)(exp(((double)thr_val - (double)tmax) * inv_t) * 1099511627776.0);
        const unsigned long long need = target > above ? target - above : 1ull;
        ties_keep = w ? (int32_t)min((unsigned long long)0x7fffffff, (need + w - 1) / w) : 1;
        if (ties_keep < 1) ties_keep = 1;
    }

    if (single) {
        token = targ;
        kept = 1.0;   // exp(0) of the arg-max: the mass of a one-token nucleus
    } else {
        const int chunk = (V + kThreads - 1) / kThreads;
        const int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);
        int32_t rank = 0;
        if (nucleus) {
            int32_t my_ties = 0;
            for (int i = c0; i < c1; ++i) my_ties += order_key(l[i]) == thr;
            rank = block_exclusive_scan_int(sh, my_ties, nullptr);
        }
        const int32_t rank0 = rank;
        double mine = 0.0;
        int32_t my_last = -1;
        for (int i = c0; i < c1; ++i) {
            const float v = l[i];
            bool keep = true;
            if (nucleus) {
                const uint32_t key = order_key(v);
                keep = key > thr || (key == thr && rank < ties_keep);
                if (key == thr) ++rank;
            }
            if (keep) {
                const double p = exp(((double)v - (double)tmax) * inv_t);
                if (p > 0.0) { mine += p; my_last = i; }
            } else if (v2) {
                l[i] = -INFINITY;   // v2 reports under the truncated distribution
            }
        }
        double kept_total;
        const double base = block_exclusive_scan(sh, mine, &kept_total);
        kept = kept_total;
        const double draw = philox_uniform(d.seed, d.draw_lo, d.draw_hi) * kept;
        if (tid == 0) { sh.ival2 = -1; }
        __syncthreads();
        if (mine > 0.0 && draw >= base && draw < base + mine) {
            double acc = base;
            int32_t pick = my_last;
            rank = rank0;
            for (int i = c0; i < c1; ++i) {
                const float v = l[i];
                bool keep = true;
                if (nucleus && !v2) {
                    const uint32_t key = order_key(v);
                    keep = key > thr || (key == thr && rank < ties_keep);
                    if (key == thr) ++rank;
                }
                if (!keep) continue;
                const double p = exp(((double)v - (double)tmax) * inv_t);
                if (p <= 0.0) continue;
                acc += p;
                if (draw < acc) { pick = i; break; }
            }
            sh.ival2 = pick;
        }
        __syncthreads();
        if (sh.ival2 < 0) {
            // rounding left the draw past the last boundary: the last kept token
            float dummy;
            int32_t last;
            block_argmax(sh, (float)my_last, -my_last, dummy, last);
            token = (int32_t)dummy;
        } else {
            token = sh.ival2;
        }
    }

    // ---- outputs
    __syncthreads();
    // A row whose reasoning budget is forcing reports the forced token in place of the drawn one (the draw still
    // happened: the request's counter moves as in the reference, which samples first and replaces afterwards).
    const int32_t drawn = token;
    const bool forced = d.pad[1] != 0;
    if (forced) token = (int32_t)d.pad[1] - 1;
    if (v2 && n_top > 0) {
        // post-transformation top-k: by probability desc (= transformed logit desc), id asc
        float pv = INFINITY;
        int32_t pid = -1;
        for (uint32_t j = 0; j < n_top; ++j) {
            float bv = -INFINITY;
            int32_t bi = 0x7fffffff;
            for (int i = tid; i < V; i += kThreads) {
                float v = l[i];
                if (single && i != drawn) v = -INFINITY;
                const bool after = v < pv || (v == pv && i > pid);
                if (after && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
            }
            block_argmax(sh, bv, bi, bv, bi);
            if (tid == 0) {
                top_ids[(size_t)row * top_stride + j] = bi;
                top_lps[(size_t)row * top_stride + j] = (float)log(exp(((double)bv - (double)tmax) * inv_t) / kept);
            }
            pv = bv;
            pid = bi;
        }
    }
    if (token < 0 || token >= V) token = 0;      // a row of NaNs has no arg-max: stay inside the row
    if (tid == 0) {
        SampleOut o;
        o.token = token;
        o.logprob = (float)((double)raw[token] - (double)rmax - rlog);
        o.sampled_logprob = 0.f;
        if (v2 && (d.flags & kFlagWantLogprob)) {
            // (a one-token nucleus gives every other token, a forced one included, probability zero)
            o.sampled_logprob = single && token != drawn ? -INFINITY : (float)log(exp(((double)l[token] - (double)tmax) * inv_t) / kept);
        }
        o.n_top = n_top;
        outs[row] = o;
    }
}


// ---- greedy rows without logit edits (v2, top_k == 1): the token is the arg-max of the raw row and
// the only statistics needed are the row's maximum and its double-precision sum of exponentials.
// The row is cut into chunks of kChunk logits handled by separate blocks, so a handful of rows still
// fills the GPU; a second tiny kernel merges the chunk results in chunk order.
constexpr int kChunk = 4096, kChunkThreads = 256;

struct ChunkStat {
    double sum;      // sum of exp(l - max) over the chunk, fixed order
    float max;
    int32_t arg;     // lowest id holding the maximum
};
static_assert(sizeof(ChunkStat) == 16, "ChunkStat layout");

__global__ void __launch_bounds__(kChunkThreads) greedy_chunk_kernel(const float * __restrict__ raw_logits, int V, const SampleDesc * __restrict__ descs,
                                                                     ChunkStat * __restrict__ stats, int n_chunks) {
    const int row = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (!(descs[row].flags & kFlagGreedyFast)) return;
    __shared__ float s_max[kChunkThreads / 32];
    __shared__ int32_t s_arg[kChunkThreads / 32];
    __shared__ double s_sum[kChunkThreads / 32];
    const float * l = raw_logits + (size_t)row * V;
    const int base = chunk * kChunk;
    float v[kChunk / kChunkThreads];
    float m = -INFINITY;
    int32_t a = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kChunk / kChunkThreads; ++j) {
        const int i = base + j * kChunkThreads + tid;
        v[j] = i < V ? l[i] : -INFINITY;
        if (v[j] > m) { m = v[j]; a = i; }       // ascending ids: the first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o);
        const int32_t oa = __shfl_xor_sync(0xffffffffu, a, o);
        if (om > m || (om == m && oa < a)) { m = om; a = oa; }
    }
    if (lane == 0) { s_max[wid] = m; s_arg[wid] = a; }
    __syncthreads();
    m = s_max[0];
    a = s_arg[0];
#pragma unroll
    for (int w = 1; w < kChunkThreads / 32; ++w)
        if (s_max[w] > m || (s_max[w] == m && s_arg[w] < a)) { m = s_max[w]; a = s_arg[w]; }
    double part = 0.0;
#pragma unroll
    for (int j = 0; j < kChunk / kChunkThreads; ++j) {
        const int i = base + j * kChunkThreads + tid;
        if (i < V) part += exp((double)v[j] - (double)m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) s_sum[wid] = part;
    __syncthreads();
    if (tid == 0) {
        double sum = 0.0;
#pragma unroll
        for (int w = 0; w < kChunkThreads / 32; ++w) sum += s_sum[w];
        ChunkStat st;
        st.sum = sum;
        st.max = m;
        st.arg = a;
        stats[(size_t)row * n_chunks + chunk] = st;
    }
}

__global__ void greedy_finish_kernel(const float * __restrict__ raw_logits, int V, const SampleDesc * __restrict__ descs,
                                     const ChunkStat * __restrict__ stats, int n_chunks, SampleOut * __restrict__ outs,
                                     int32_t * __restrict__ top_ids, float * __restrict__ top_lps, int top_stride) {
    const int row = blockIdx.x;
    const SampleDesc d = descs[row];
    if (!(d.flags & kFlagGreedyFast) || threadIdx.x != 0) return;
    const ChunkStat * st = stats + (size_t)row * n_chunks;
    float rmax = st[0].max;
    int32_t token = st[0].arg;
    for (int c = 1; c < n_chunks; ++c)
        if (st[c].max > rmax) { rmax = st[c].max; token = st[c].arg; }      // chunks ascend in id: strict > keeps the lowest id
    double total = 0.0;
    for (int c = 0; c < n_chunks; ++c) total += st[c].sum * exp((double)st[c].max - (double)rmax);
    const double rlog = log(total);
    if (token < 0 || token >= V) token = 0;      // a row of NaNs has no arg-max: stay inside the row
    const float * raw = raw_logits + (size_t)row * V;
    const double inv_t = 1.0 / (double)d.temperature;
    // the one-token nucleus: its post-transformation logprob is log(exp(0 / T) / 1)
    const float self_lp = (float)log(exp(((double)raw[token] - (double)rmax) * inv_t) / 1.0);
    const uint32_t n_top = min(d.n_top, (uint32_t)min(top_stride, V));
    int32_t next_id = 0;
    for (uint32_t j = 0; j < n_top; ++j) {
        if (j == 0) {
            top_ids[(size_t)row * top_stride] = token;
            top_lps[(size_t)row * top_stride] = self_lp;
        } else {
            // every other token was truncated away: ids in ascending order, probability zero
            if (next_id == token) ++next_id;
            top_ids[(size_t)row * top_stride + j] = next_id++;
            top_lps[(size_t)row * top_stride + j] = (float)log(exp(-INFINITY * inv_t) / 1.0);
        }
    }
    SampleOut o;
    o.token = token;
    o.logprob = (float)((double)raw[token] - (double)rmax - rlog);
    o.sampled_logprob = (d.flags & kFlagWantLogprob) ? self_lp : 0.f;
    o.n_top = n_top;
    outs[row] = o;
}

} // namespace

size_t sample_scratch_bytes(int n_vocab, int n_rows) { return (size_t)n_rows * ((n_vocab + kChunk - 1) / kChunk) * sizeof(ChunkStat); }

void launch_sample(const float * raw_logits, float * work_logits, int n_vocab, int n_rows, const SampleDesc * desc, const LogitEdit * edits,
                   const uint32_t * masks, SampleOut * out,
                   int32_t * top_ids, float * top_logprobs, int top_stride, int n_greedy_fast, void * scratch, cudaStream_t stream) {
    if (n_rows <= 0) return;
    if (n_greedy_fast < n_rows)
        sample_kernel<<<n_rows, kThreads, 0, stream>>>(raw_logits, work_logits, n_vocab, desc, edits, masks, out, top_ids, top_logprobs, top_stride);
    if (n_greedy_fast > 0) {
        const int n_chunks = (n_vocab + kChunk - 1) / kChunk;
        ChunkStat * stats = static_cast<ChunkStat *>(scratch);
        greedy_chunk_kernel<<<dim3(n_chunks, n_rows), kChunkThreads, 0, stream>>>(raw_logits, n_vocab, desc, stats, n_chunks);
        greedy_finish_kernel<<<n_rows, 32, 0, stream>>>(raw_logits, n_vocab, desc, stats, n_chunks, out, top_ids, top_logprobs, top_stride);
    }
}

} // namespace rb200
