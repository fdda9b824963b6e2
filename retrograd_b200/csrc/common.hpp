// Shared host-side plumbing: status codes, the thread-local error slot and the exception fence
// every C entry point runs behind (the reference's convention:
// crates/retrograd-ffi/runtime/include/retro_lora_train.h:2701-2706,3038 and
// crates/retrograd-ffi/runtime/src/retro_runtime.hpp:37,1255-1267).
#pragma once

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

namespace rb200 {

constexpr int STATUS_OK = 0;
constexpr int STATUS_RUNTIME = -1;
constexpr int STATUS_BUFFER_TOO_SMALL = -2;
constexpr int STATUS_INVALID_ARGUMENT = -3;

std::string & last_error();
inline void set_error(const std::string & message) { last_error() = message; }
inline void clear_error() { last_error().clear(); }

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

#define RB_CUDA(expr)                                                                              \
    do {                                                                                           \
        cudaError_t rb_status_ = (expr);                                                           \
        if (rb_status_ != cudaSuccess) {                                                           \
            throw ::rb200::CudaError(std::string("CUDA error: ") + cudaGetErrorString(rb_status_) + \
                                     " at " + __FILE__ + ":" + std::to_string(__LINE__));          \
        }                                                                                          \
    } while (0)

template <class F> int boundary(F && body) {
    try {
        clear_error();
        return body();
    } catch (const std::exception & err) {
        set_error(err.what());
        return STATUS_RUNTIME;
    } catch (...) {
        set_error("unknown C++ exception");
        return STATUS_RUNTIME;
    }
}

} // namespace rb200
