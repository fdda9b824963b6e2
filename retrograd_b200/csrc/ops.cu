// Operator-level entry points: one kernel of the decode step run on caller-provided host data.
// They exist so a kernel can be checked against the CPU oracle and timed in isolation (small
// cases for profiler captures) without building a model around it.

#include "engine.hpp"
#include "blocks.hpp"

#include <vector>

using namespace rb200;

extern "C" {

// y[t][o] = sum_k deq(w)[o][k] x[t][k]. `path`: 0 = what the engine would pick, 1 = f32 row kernel,
// 3 = exact tensor-core kernel (mma.sync), 4 = exact tcgen05 kernel, 5 = exact weight-streaming kernel (at most 8 tokens). The kernel runs `iters`
// times; *out_ms receives the mean device time per launch (CUDA events on the launching stream).
int retro_b200_op_gemm(uint32_t ggml_type, const uint8_t * w, uint32_t n_out, uint32_t n_in, const float * x, uint32_t n_tokens, float * y,
                       int path, uint32_t iters, float * out_ms) {
    return boundary([&]() -> int {
        const size_t rb = row_bytes(ggml_type, n_in);
        if (!w || !x || !y || rb == 0 || n_in % 8 != 0 || n_tokens == 0 || n_out == 0) {
            set_error("op_gemm: bad arguments");
            return STATUS_INVALID_ARGUMENT;
        }
        DeviceBuffer<uint8_t> dw;
        DeviceBuffer<float> dx, dy;
        SplitBuffer xs;
        dw.ensure(rb * n_out);
        dx.ensure((size_t)n_tokens * n_in);
        dy.ensure((size_t)n_tokens * n_out);
        xs.ensure(n_tokens, n_in);
        cudaStream_t stream;
        RB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        cudaEvent_t e0, e1;
        RB_CUDA(cudaEventCreate(&e0));
        RB_CUDA(cudaEventCreate(&e1));
        RB_CUDA(cudaMemcpyAsync(dw.ptr, w, rb * n_out, cudaMemcpyHostToDevice, stream));
        RB_CUDA(cudaMemcpyAsync(dx.ptr, x, (size_t)n_tokens * n_in * 4, cudaMemcpyHostToDevice, stream));
        WeightView wv;
        wv.data = dw.ptr;
        wv.type = ggml_type;
        wv.n_in = n_in;
        wv.n_out = n_out;
        wv.row_bytes = (uint32_t)rb;
        DeviceBuffer<uint8_t> dtiled;
        if (ggml_type == GGML_Q4_K && n_in % 256 == 0 && (path == 4 || path == 5 || path == 0)) {
            dtiled.ensure(q4k_tiled_bytes(n_out, n_in));
            launch_q4k_retile(dw.ptr, n_out, n_in, (uint32_t)rb, dtiled.ptr, stream);
            wv.tiled = dtiled.ptr;
            wv.tc5_exact = q4k_min_fold_ok(w, (size_t)n_out * (n_in / 256));
        }
        if (ggml_type == GGML_Q8_0 && n_in % 256 == 0 && path == 5) {
            dtiled.ensure(q8_0_tiled_bytes(n_out, n_in));
            launch_q8_0_retile(dw.ptr, n_out, n_in, (uint32_t)rb, dtiled.ptr, stream);
            wv.tiled = dtiled.ptr;
        }
        if (ggml_type == GGML_Q8_0 && n_in % 64 == 0) wv.tc5_exact = q8_0_products_fit_f16(w, (size_t)n_out * (n_in / 32));
        const bool have_split = xs.get() != nullptr;
        if (have_split) launch_split_prep(dx.ptr, (int)n_in, (int)n_in, (int)n_tokens, xs.view, stream);
        int chosen = path;
        if (chosen == 0) chosen = have_split && n_tokens > 64 && gemm_q4k_tc5_supported(wv, xs.view) ? 4 : have_split && n_tokens > 8 && gemm_q4k_exact_supported(wv, xs.view) ? 3 : 1;
        DeviceBuffer<float> tc5_scratch;
        DeviceBuffer<int> flag;
        flag.ensure(1);
        RB_CUDA(cudaMemsetAsync(flag.ptr, 0, sizeof(int), stream));
        DeviceBuffer<float> stream_scratch;
        int n_sm = 148;
        {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        }
        if (chosen == 5) {
            if (!(have_split && (gemm_q4k_stream_supported(wv, xs.view, (int)n_tokens) || gemm_q8_0_stream_supported(wv, xs.view, (int)n_tokens)))) {
                cudaStreamDestroy(stream);
                set_error("op_gemm: the requested kernel does not cover this type or shape");
                return STATUS_INVALID_ARGUMENT;
            }
            stream_scratch.ensure(gemm_q4k_stream_scratch_floats(n_out, n_in));
        }
        if (chosen == 4 && ggml_type == GGML_Q4_K) {
            const size_t need = gemm_q4k_tc5_scratch_floats(wv.n_out, wv.n_in, (int)n_tokens, n_sm);
            if (need) tc5_scratch.ensure(need);
        }
        if (chosen == 4 && !(have_split && (gemm_q4k_tc5_supported(wv, xs.view) || gemm_q8_0_tc5_supported(wv, xs.view)))) {
            cudaStreamDestroy(stream);
            set_error("op_gemm: the requested kernel does not cover this type or shape");
            return STATUS_INVALID_ARGUMENT;
        }
        if ((chosen == 3 && !(have_split && (gemm_q4k_exact_supported(wv, xs.view) || gemm_q8_0_exact_supported(wv, xs.view)))) || chosen == 2) {
            cudaStreamDestroy(stream);
            set_error("op_gemm: the requested kernel does not cover this type or shape");
            return STATUS_INVALID_ARGUMENT;
        }
        auto run = [&]() {
            if (chosen == 5 && ggml_type == GGML_Q8_0) launch_gemm_q8_0_stream(wv, xs.view, (int)n_tokens, dy.ptr, (int)n_out, nullptr, nullptr, 0, stream_scratch.ptr, n_sm, flag.ptr, stream);
            else if (chosen == 5) launch_gemm_q4k_stream(wv, xs.view, (int)n_tokens, dy.ptr, (int)n_out, nullptr, nullptr, 0, stream_scratch.ptr, n_sm, flag.ptr, stream);
            else if (chosen == 4 && ggml_type == GGML_Q8_0) launch_gemm_q8_0_tc5(wv, xs.view, (int)n_tokens, dy.ptr, (int)n_out, nullptr, nullptr, 0, flag.ptr, n_sm, stream);
            else if (chosen == 4) launch_gemm_q4k_tc5(wv, xs.view, (int)n_tokens, dy.ptr, (int)n_out, nullptr, nullptr, 0, flag.ptr, tc5_scratch.ptr, tc5_scratch.count, n_sm, stream);
            else if (chosen == 3 && ggml_type == GGML_Q8_0) launch_gemm_q8_0_exact(wv, xs.view, (int)n_tokens, dy.ptr, (int)n_out, nullptr, nullptr, 0, stream);
            else if (chosen == 3) launch_gemm_q4k_exact(wv, xs.view, (int)n_tokens, dy.ptr, (int)n_out, nullptr, nullptr, 0, stream);
            else launch_gemm_rows(wv, dx.ptr, (int)n_in, (int)n_tokens, dy.ptr, (int)n_out, nullptr, nullptr, 0, stream);
        };
        run();   // warm-up, also the launch whose output is returned
        // Operands that fit in L2 would be re-read from it by back-to-back launches: then every timed
        // launch is preceded by a write of a buffer larger than L2 and timed with its own event pair.
        const size_t operand_bytes = (size_t)row_bytes(ggml_type, n_in) * n_out + (size_t)n_tokens * n_in * 4;
        const bool flush = iters > 0 && operand_bytes < ((size_t)256 << 20);
        DeviceBuffer<uint8_t> flush_buf;
        std::vector<cudaEvent_t> marks;
        if (flush) {
            flush_buf.ensure((size_t)256 << 20);
            marks.resize(2 * (size_t)iters);
            for (auto & m : marks) RB_CUDA(cudaEventCreate(&m));
        }
        RB_CUDA(cudaEventRecord(e0, stream));
        for (uint32_t i = 0; i < iters; ++i) {
            if (flush) {
                RB_CUDA(cudaMemsetAsync(flush_buf.ptr, (int)i, (size_t)256 << 20, stream));
                RB_CUDA(cudaEventRecord(marks[2 * i], stream));
            }
            run();
            if (flush) RB_CUDA(cudaEventRecord(marks[2 * i + 1], stream));
        }
        RB_CUDA(cudaEventRecord(e1, stream));
        RB_CUDA(cudaMemcpyAsync(y, dy.ptr, (size_t)n_tokens * n_out * 4, cudaMemcpyDeviceToHost, stream));
        int h_flag = 0;
        RB_CUDA(cudaMemcpyAsync(&h_flag, flag.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream));
        RB_CUDA(cudaStreamSynchronize(stream));
        RB_CUDA(cudaGetLastError());
        if (h_flag) {
            cudaStreamDestroy(stream);
            set_error("op_gemm: a pipeline wait inside the tensor-core kernel timed out");
            return STATUS_RUNTIME;
        }
        float ms = 0.f;
        if (iters) cudaEventElapsedTime(&ms, e0, e1);
        if (flush) {
            ms = 0.f;
            for (uint32_t i = 0; i < iters; ++i) {
                float one = 0.f;
                cudaEventElapsedTime(&one, marks[2 * i], marks[2 * i + 1]);
                ms += one;
            }
            for (auto & m : marks) cudaEventDestroy(m);
        }
        if (out_ms) *out_ms = iters ? ms / iters : 0.f;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        cudaStreamDestroy(stream);
        return STATUS_OK;
    });
}

// The grouped MXFP4 expert GEMM on tcgen05: `banks` holds n_expert matrices of n_out rows x n_in MXFP4 weights
// (17-byte blocks, rows consecutive), x the n_rows = offsets[n_expert] activation rows sorted by expert, offsets
// each expert's first row. y[r][o] = sum_k deq(bank[e(r)])[o][k] x[r][k]. `iters` further launches are timed
// (CUDA events on the launching stream, L2 flushed before each); *out_ms is their mean.
int retro_b200_op_gemm_mxfp4_grouped(const uint8_t * banks, uint32_t n_expert, uint32_t n_out, uint32_t n_in, const float * x,
                                     const int32_t * offsets, float * y, uint32_t iters, float * out_ms) {
    return boundary([&]() -> int {
        if (!banks || !x || !y || !offsets || n_expert == 0 || n_out == 0 || n_in == 0 || n_in % 64 != 0) {
            set_error("op_gemm_mxfp4_grouped: bad arguments");
            return STATUS_INVALID_ARGUMENT;
        }
        const int n_rows = offsets[n_expert];
        const size_t bank_bytes = (size_t)n_expert * n_out * (n_in / 32) * 17;
        if (n_rows <= 0 || !tensor_maps_available() || !mxfp4_scales_are_f16(banks, bank_bytes / 17)) {
            set_error("op_gemm_mxfp4_grouped: the kernel does not cover these operands");
            return STATUS_INVALID_ARGUMENT;
        }
        DeviceBuffer<uint8_t> d_bank, d_tiled;
        DeviceBuffer<float> dx, dy;
        DeviceBuffer<int32_t> d_off;
        DeviceBuffer<int> flag;
        SplitBuffer xs;
        d_bank.ensure(bank_bytes);
        d_tiled.ensure(mxfp4_tiled_bytes(n_expert, n_out, n_in));
        dx.ensure((size_t)n_rows * n_in);
        dy.ensure((size_t)n_rows * n_out);
        d_off.ensure(n_expert + 1);
        flag.ensure(1);
        xs.ensure((size_t)n_rows, n_in);
        cudaStream_t stream;
        RB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        RB_CUDA(cudaMemcpyAsync(d_bank.ptr, banks, bank_bytes, cudaMemcpyHostToDevice, stream));
        RB_CUDA(cudaMemcpyAsync(dx.ptr, x, (size_t)n_rows * n_in * 4, cudaMemcpyHostToDevice, stream));
        RB_CUDA(cudaMemcpyAsync(d_off.ptr, offsets, (n_expert + 1) * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
        RB_CUDA(cudaMemsetAsync(flag.ptr, 0, sizeof(int), stream));
        RB_CUDA(cudaMemsetAsync(dy.ptr, 0, (size_t)n_rows * n_out * 4, stream));
        launch_mxfp4_retile(d_bank.ptr, n_expert, n_out, n_in, d_tiled.ptr, stream);
        launch_split_prep(dx.ptr, (int)n_in, (int)n_in, n_rows, xs.view, stream);
        WeightView wv;
        wv.type = GGML_MXFP4;
        wv.n_in = n_in;
        wv.n_out = n_out;
        wv.row_bytes = (n_in / 32) * 17;
        wv.tiled = d_tiled.ptr;
        if (!gemm_mxfp4_tc5_supported(wv, xs.view)) {
            cudaStreamDestroy(stream);
            set_error("op_gemm_mxfp4_grouped: the kernel does not cover these operands");
            return STATUS_INVALID_ARGUMENT;
        }
        launch_gemm_mxfp4_tc5_grouped(wv, (int)n_expert, d_off.ptr, xs.view, n_rows, dy.ptr, (int)n_out, flag.ptr, stream);
        // `iters` timed launches, each behind a write of a buffer larger than L2
        float total_ms = 0.f;
        if (iters) {
            DeviceBuffer<uint8_t> flush_buf;
            flush_buf.ensure((size_t)256 << 20);
            cudaEvent_t e0, e1;
            RB_CUDA(cudaEventCreate(&e0));
            RB_CUDA(cudaEventCreate(&e1));
            for (uint32_t i = 0; i < iters; ++i) {
                RB_CUDA(cudaMemsetAsync(flush_buf.ptr, (int)i, (size_t)256 << 20, stream));
                RB_CUDA(cudaEventRecord(e0, stream));
                launch_gemm_mxfp4_tc5_grouped(wv, (int)n_expert, d_off.ptr, xs.view, n_rows, dy.ptr, (int)n_out, flag.ptr, stream);
                RB_CUDA(cudaEventRecord(e1, stream));
                RB_CUDA(cudaStreamSynchronize(stream));
                float one = 0.f;
                cudaEventElapsedTime(&one, e0, e1);
                total_ms += one;
            }
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
        }
        if (out_ms) *out_ms = iters ? total_ms / iters : 0.f;
        int h_flag = 0;
        RB_CUDA(cudaMemcpyAsync(y, dy.ptr, (size_t)n_rows * n_out * 4, cudaMemcpyDeviceToHost, stream));
        RB_CUDA(cudaMemcpyAsync(&h_flag, flag.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream));
        RB_CUDA(cudaStreamSynchronize(stream));
        RB_CUDA(cudaGetLastError());
        cudaStreamDestroy(stream);
        if (h_flag) {
            set_error("op_gemm_mxfp4_grouped: a pipeline wait inside the tensor-core kernel timed out");
            return STATUS_RUNTIME;
        }
        return STATUS_OK;
    });
}

} // extern "C"
