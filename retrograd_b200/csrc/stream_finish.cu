// Finish kernels of the split-K GEMMs (the weight-streaming kernels and the tcgen05 kernel's split form):
// they add the K chunks' partial sums in chunk order, add bias and residual, and optionally run the
// layer's next row-wise step (RMS norm, or SwiGLU of a [gate | up] row) on the row while it is in
// registers, writing the split form the next GEMM reads.

#include "kernels.cuh"
#include "split_emit.cuh"

namespace rb200 {

namespace {

// The chunks' partial sums of one result, added in chunk order. The loads of up to eight chunks are
// issued before the first addition, so the kernel pays one memory latency instead of one per chunk.
__device__ __forceinline__ float sum_chunks1(const float * __restrict__ partial, int n_chunks, size_t chunk_stride, size_t at) {
    float s = 0.f;
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {
        float p[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) p[c] = c0 + c < n_chunks ? partial[(size_t)(c0 + c) * chunk_stride + at] : 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            if (c0 + c < n_chunks) s += p[c];
    }
    return s;
}

__device__ __forceinline__ float4 sum_chunks4(const float * __restrict__ partial, int n_chunks, int n_out, int t_stride, int t, int o) {
    const size_t chunk_stride = (size_t)t_stride * n_out, at = (size_t)t * n_out + o;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {
        float4 p[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
            p[c] = c0 + c < n_chunks ? *reinterpret_cast<const float4 *>(partial + (size_t)(c0 + c) * chunk_stride + at) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (c0 + c < n_chunks) { s.x += p[c].x; s.y += p[c].y; s.z += p[c].z; s.w += p[c].w; }
        }
    }
    return s;
}

// y[t][o] = sum over K chunks (in order) of partial + bias + residual
__global__ void stream_finish_kernel(const float * __restrict__ partial, int n_chunks, int n_out, int T, int t_stride, float * __restrict__ y, int ldy,
                                     const float * __restrict__ bias, const float * __restrict__ residual, int ldr) {
    pdl_trigger();
    pdl_wait();
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (o >= n_out || t >= T) return;
    float sum = sum_chunks1(partial, n_chunks, (size_t)t_stride * n_out, (size_t)t * n_out + o);
    if (bias) sum += bias[o];
    if (residual) sum += residual[(size_t)t * ldr + o];
    y[(size_t)t * ldy + o] = sum;
}

// One CTA of 1024 threads per token: the row sum (as above, written to y, which may alias the
// residual), then the RMS norm of the row. The sum of squares is added in the order of the separate
// norm kernel (256 threads, four columns each, strided by 1024 columns): thread q's columns belong to
// that kernel's thread q % 256, whose terms are added in ascending column order through shared memory.
__global__ void __launch_bounds__(1024) stream_finish_norm_kernel(const float * __restrict__ partial, int n_chunks, int n_out, int t_stride, float * y,
                                                                  int ldy, const float * __restrict__ bias, const float * residual, int ldr,
                                                                  const float * __restrict__ norm_w, float eps, float * __restrict__ out, int ld_out,
                                                                  SplitAct split) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sq[1024];
    __shared__ float red[32];
    const int t = blockIdx.x;
    float * yr = y + (size_t)t * ldy;
    float ss = 0.f;         // meaningful in threads 0..255
    for (int base = 0; base < n_out; base += 4096) {
        const int i = base + threadIdx.x * 4;
        float term = 0.f;
        if (i < n_out) {
            float4 v = sum_chunks4(partial, n_chunks, n_out, t_stride, t, i);
            if (bias) {
                const float4 b = *reinterpret_cast<const float4 *>(bias + i);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            if (residual) {
                const float4 r = *reinterpret_cast<const float4 *>(residual + (size_t)t * ldr + i);
                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            }
            *reinterpret_cast<float4 *>(yr + i) = v;
            term = (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
        sq[threadIdx.x] = term;
        __syncthreads();
        if (threadIdx.x < 256) {
#pragma unroll
            for (int m = 0; m < 4; ++m)
                if (base + m * 1024 + threadIdx.x * 4 < n_out) ss += sq[m * 256 + threadIdx.x];
        }
        __syncthreads();
    }
    if (threadIdx.x < 256) {
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    const float scale = 1.0f / sqrtf(red[0] / (float)n_out + eps);
    for (int base = 0; base < n_out; base += 4096) {
        const int i = base + threadIdx.x * 4;
        const bool active = i < n_out;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (active) {
            // the thread reads back the columns it wrote itself
            const float4 a = *reinterpret_cast<const float4 *>(yr + i), b = *reinterpret_cast<const float4 *>(norm_w + i);
            v = make_float4(a.x * scale * b.x, a.y * scale * b.y, a.z * scale * b.z, a.w * scale * b.w);
            if (out) *reinterpret_cast<float4 *>(out + (size_t)t * ld_out + i) = v;
        }
        if (split.hi) emit_split4(split, t, i, v, active);
    }
}

// Grid (ceil(ff / 1024), tokens): column i of the gate half and of the up half of the row are summed
// (with their bias), then h = silu(gate) * up in the arithmetic of the separate SwiGLU kernel.
__global__ void __launch_bounds__(256) stream_finish_swiglu_kernel(const float * __restrict__ partial, int n_chunks, int n_out, int t_stride,
                                                                   const float * __restrict__ bias, float * __restrict__ out, int ld_out,
                                                                   SplitAct split) {
    pdl_trigger();
    pdl_wait();
    const int ff = n_out >> 1;
    const int t = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const bool active = i < ff;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
        float4 g = sum_chunks4(partial, n_chunks, n_out, t_stride, t, i), u = sum_chunks4(partial, n_chunks, n_out, t_stride, t, ff + i);
        if (bias) {
            const float4 bg = *reinterpret_cast<const float4 *>(bias + i), bu = *reinterpret_cast<const float4 *>(bias + ff + i);
            g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w;
            u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
        }
        v = make_float4(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y, g.z / (1.0f + expf(-g.z)) * u.z,
                        g.w / (1.0f + expf(-g.w)) * u.w);
        if (out) *reinterpret_cast<float4 *>(out + (size_t)t * ld_out + i) = v;
    }
    if (split.hi) emit_split4(split, t, i, v, active);
}

bool aligned16(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

} // namespace

bool finish_tail_supported(const FinishTail & tail, int n_out, const float * y, int ldy, const float * bias, const float * residual, int ldr) {
    if (tail.kind == 3) return tail.rope && !residual && rope_store_from_partial_supported(*tail.rope, y, ldy, n_out, bias);
    if (!tail.out && !tail.split.hi) return false;
    if (bias && !aligned16(bias)) return false;
    if (tail.out && (!aligned16(tail.out) || tail.ld_out % 4 != 0)) return false;
    if (tail.kind == 1) {
        return n_out % 32 == 0 && tail.norm_w && aligned16(tail.norm_w) && aligned16(y) && ldy % 4 == 0 && tail.out != y &&
               (!residual || (aligned16(residual) && ldr % 4 == 0)) && (!tail.split.hi || tail.split.ld == n_out);
    }
    if (tail.kind == 2) return n_out % 64 == 0 && !residual && (!tail.split.hi || tail.split.ld == n_out / 2);
    return false;
}

void launch_gemm_stream_finish(const float * scratch, int n_chunks, int n_out, int n_tokens, int t_stride, float * y, int ldy, const float * bias,
                               const float * residual, int ldr, cudaStream_t stream, const FinishTail * tail) {
    if (tail && tail->kind == 1) {
        launch_pdl(stream_finish_norm_kernel, dim3(n_tokens), dim3(1024), 0, stream, scratch, n_chunks, n_out, t_stride, y, ldy, bias, residual, ldr,
                   tail->norm_w, tail->eps, tail->out, tail->ld_out, tail->split);
    } else if (tail && tail->kind == 3) {
        launch_rope_store(y, ldy, n_tokens, *tail->rope, stream, scratch, n_chunks, t_stride, n_out, bias);
    } else if (tail && tail->kind == 2) {
        launch_pdl(stream_finish_swiglu_kernel, dim3((n_out / 2 + 1023) / 1024, n_tokens), dim3(256), 0, stream, scratch, n_chunks, n_out, t_stride, bias,
                   tail->out, tail->ld_out, tail->split);
    } else {
        launch_pdl(stream_finish_kernel, dim3((n_out + 255) / 256, n_tokens), dim3(256), 0, stream, scratch, n_chunks, n_out, n_tokens, t_stride, y, ldy,
                   bias, residual, ldr);
    }
}

} // namespace rb200
