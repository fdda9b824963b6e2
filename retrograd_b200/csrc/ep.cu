// Expert-parallel support: the exchange plan, the run-time NCCL binding and the row gather / scatter
// kernels around the all-to-all. See ep.hpp.

#include "ep.hpp"
#include "kernels.cuh"

#include <dlfcn.h>

#include <mutex>
#include <stdexcept>

namespace rb200 {

void ep_make_plan(const int32_t * all_offsets, int world, int rank, int n_expert, EpPlan & plan) {
    const int per = n_expert / world;
    const int stride = n_expert + 1;
    const int32_t * mine = all_offsets + (size_t)rank * stride;
    plan.send_begin.assign(world, 0);
    plan.send_count.assign(world, 0);
    plan.recv_begin.assign(world, 0);
    plan.recv_count.assign(world, 0);
    int32_t at = 0;
    for (int p = 0; p < world; ++p) {
        // my pairs for p's experts are one contiguous range of my expert-sorted pairs
        plan.send_begin[p] = mine[p * per];
        plan.send_count[p] = mine[(p + 1) * per] - mine[p * per];
        const int32_t * theirs = all_offsets + (size_t)p * stride;
        plan.recv_begin[p] = at;
        plan.recv_count[p] = theirs[(rank + 1) * per] - theirs[rank * per];
        at += plan.recv_count[p];
    }
    plan.n_recv = at;
    plan.offsets.assign(n_expert + 1, 0);
    plan.sorted.clear();
    plan.sorted.reserve(at);
    for (int e = 0; e < n_expert; ++e) {
        plan.offsets[e] = (int32_t)plan.sorted.size();
        if (e / per != rank) continue;
        for (int p = 0; p < world; ++p) {
            const int32_t * theirs = all_offsets + (size_t)p * stride;
            // p's pairs of expert e sit behind p's pairs of my earlier experts inside p's block of the receive buffer
            const int32_t first = plan.recv_begin[p] + (theirs[e] - theirs[rank * per]);
            for (int32_t j = 0; j < theirs[e + 1] - theirs[e]; ++j) plan.sorted.push_back(first + j);
        }
    }
    plan.offsets[n_expert] = (int32_t)plan.sorted.size();
}

const NcclApi & nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    static std::string failure;
    std::call_once(once, [] {
        // the copy already mapped into the process (same soname) is returned if there is one
        void * lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) {
            failure = std::string("expert parallelism needs NCCL: ") + dlerror();
            return;
        }
        api.lib = lib;
        auto need = [&](const char * name) -> void * {
            void * sym = dlsym(lib, name);
            if (!sym && failure.empty()) failure = std::string("expert parallelism needs NCCL: symbol ") + name + " is missing";
            return sym;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(need("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(need("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(need("ncclCommDestroy"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(need("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(need("ncclGroupEnd"));
        api.Send = reinterpret_cast<decltype(api.Send)>(need("ncclSend"));
        api.Recv = reinterpret_cast<decltype(api.Recv)>(need("ncclRecv"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(need("ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(need("ncclGetErrorString"));
    });
    if (!failure.empty()) throw std::runtime_error(failure);
    return api;
}

namespace {

__global__ void ep_gather_rows_kernel(const float * __restrict__ x, int ldx, const int32_t * __restrict__ sorted, int x_div, int d,
                                      float * __restrict__ out) {
    const int i = blockIdx.x;
    const float * src = x + (size_t)(sorted[i] / x_div) * ldx;
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[(size_t)i * d + c] = src[c];
}

__global__ void ep_scatter_rows_kernel(const float * __restrict__ in, const int32_t * __restrict__ sorted, int d, float * __restrict__ out, int ldo) {
    const int i = blockIdx.x;
    float * dst = out + (size_t)sorted[i] * ldo;
    for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = in[(size_t)i * d + c];
}

} // namespace

void launch_ep_gather_rows(const float * x, int ldx, const int32_t * sorted, int x_div, int n, int d, float * out, cudaStream_t stream) {
    if (n > 0) ep_gather_rows_kernel<<<n, 256, 0, stream>>>(x, ldx, sorted, x_div, d, out);
}

void launch_ep_scatter_rows(const float * in, const int32_t * sorted, int n, int d, float * out, int ldo, cudaStream_t stream) {
    if (n > 0) ep_scatter_rows_kernel<<<n, 256, 0, stream>>>(in, sorted, d, out, ldo);
}

} // namespace rb200
