// A dequant-fused Q4_K GEMM entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on their hot path: a serving process that hands
// its whole device-memory budget to its own pool at start-up and forbids later allocations, or a
// latency-critical loop that cannot afford the implicit device synchronisation an allocation or a
// free may cause. The exact tensor-core GEMM needs scratch beyond its inputs and outputs (the
// two-term f16 split of the activations and their per-sub-block sums). Here that scratch is a
// fixed array that is part of the library image: every GPU that loads the library holds it until
// the process exits, and no call of this entry point allocates or frees anything.

#include "common.hpp"
#include "kernels.cuh"
#include "blocks.hpp"

namespace rb200 {

namespace {

// Largest activation matrix the entry point accepts: n_tokens * n_in elements.
constexpr size_t kNoAllocMaxElements = (size_t)1 << 20;
constexpr size_t kHalfBytes = kNoAllocMaxElements * sizeof(__half);                // hi, and again lo
constexpr size_t kSumBytes = (kNoAllocMaxElements / 32) * sizeof(__half) + 256;    // sum_hi, and again sum_lo
constexpr size_t kScratchBytes = 2 * kHalfBytes + 2 * kSumBytes;                   // about 4.1 MiB

// In host code this name is only a handle for the runtime, not a device address: the address the
// kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char * g_scratch_of_device[kMaxDevices] = {};

// Resolves the scratch array's device address for the current device, once per device.
unsigned char * scratch_for_current_device() {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        set_error("gemm_q4k_noalloc: no current CUDA device");
        return nullptr;
    }
    if (!g_scratch_of_device[device]) {
        void * ptr = nullptr;
        const cudaError_t status = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (status != cudaSuccess || !ptr) {
            set_error(std::string("gemm_q4k_noalloc: cannot resolve the scratch array on this device: ") + cudaGetErrorString(status));
            return nullptr;
        }
        g_scratch_of_device[device] = static_cast<unsigned char *>(ptr);
    }
    return g_scratch_of_device[device];
}

} // namespace

} // namespace rb200

using namespace rb200;

extern "C" {

// y[t][o] = sum_k deq(w)[o][k] * x[t][k] with `w` stored as Q4_K rows; all three pointers are DEVICE
// pointers owned by the caller, `stream` is the caller's cudaStream_t (NULL for the default
// stream). The work is enqueued on that stream; the call does not wait for it.
//
// - Limit: n_tokens * n_in <= 1 048 576 and n_in a multiple of 256; larger shapes are refused
//   with -3 and a message, nothing is launched. d_w must be 16-byte aligned (the kernel reads
//   weight blocks as 16-byte words); a misaligned pointer is refused the same way.
// - The first call on a device resolves the scratch array's address for that device (with that
//   device current): a host-side symbol lookup, no allocation.
// - Every call on a device uses the same scratch array. Nothing in it has to start at zero: a call
//   rewrites every byte it later reads. For the same reason two calls whose work overlaps on
//   the GPU (different streams, no ordering between them) race on it - order them.
// - No cudaMalloc, cudaFree or allocating library routine is called, on any call.
int retro_b200_gemm_q4k_noalloc(const uint8_t * d_w, uint32_t n_out, uint32_t n_in, const float * d_x, uint32_t n_tokens, float * d_y,
                                void * stream) {
    return boundary([&]() -> int {
        if (!d_w || !d_x || !d_y || n_out == 0 || n_tokens == 0) {
            set_error("gemm_q4k_noalloc: device pointers and non-zero sizes are required");
            return STATUS_INVALID_ARGUMENT;
        }
        if (n_in == 0 || n_in % 256 != 0) {
            set_error("gemm_q4k_noalloc: n_in must be a multiple of 256 (whole Q4_K blocks)");
            return STATUS_INVALID_ARGUMENT;
        }
        // the kernel reads weight blocks as 16-byte words (a Q4_K block is 144 bytes, so every block of an
        // aligned matrix is aligned) and writes f32 results
        if (reinterpret_cast<uintptr_t>(d_w) % 16 != 0 || reinterpret_cast<uintptr_t>(d_x) % 4 != 0 || reinterpret_cast<uintptr_t>(d_y) % 4 != 0) {
            set_error("gemm_q4k_noalloc: d_w must be 16-byte aligned, d_x and d_y 4-byte aligned");
            return STATUS_INVALID_ARGUMENT;
        }
        if ((size_t)n_tokens * n_in > kNoAllocMaxElements) {
            set_error("gemm_q4k_noalloc: n_tokens * n_in exceeds the fixed scratch of 1048576 activation elements");
            return STATUS_INVALID_ARGUMENT;
        }
        unsigned char * scratch = scratch_for_current_device();
        if (!scratch) return STATUS_RUNTIME;
        SplitAct split;
        split.hi = reinterpret_cast<__half *>(scratch);
        split.lo = reinterpret_cast<__half *>(scratch + kHalfBytes);
        split.sum_hi = reinterpret_cast<__half *>(scratch + 2 * kHalfBytes);
        split.sum_lo = reinterpret_cast<__half *>(scratch + 2 * kHalfBytes + kSumBytes);
        split.ld = (int)n_in;
        WeightView w;
        w.data = d_w;
        w.type = GGML_Q4_K;
        w.n_in = n_in;
        w.n_out = n_out;
        w.row_bytes = (uint32_t)row_bytes(GGML_Q4_K, n_in);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        launch_split_prep(d_x, (int)n_in, (int)n_in, (int)n_tokens, split, s);
        launch_gemm_q4k_exact(w, split, (int)n_tokens, d_y, (int)n_out, nullptr, nullptr, 0, s);
        const cudaError_t status = cudaGetLastError();
        if (status != cudaSuccess) {
            set_error(std::string("gemm_q4k_noalloc: launch failed: ") + cudaGetErrorString(status));
            return STATUS_RUNTIME;
        }
        return STATUS_OK;
    });
}

} // extern "C"
