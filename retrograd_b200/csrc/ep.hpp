// Expert parallelism for MoE models: the experts are partitioned over the ranks (expert e belongs to rank
// e / (n_expert / world)), every rank runs its own requests, and per MoE layer the (token, expert)
// pairs travel to the expert's rank and back:
//   all-gather of every rank's per-expert pair offsets  ->  every rank derives the SAME exchange plan
//   dispatch (send / recv of activation rows)           ->  grouped expert GEMMs on local experts
//   combine  (send / recv of the results, reversed)     ->  weighted sum on the token's own rank
// Per-pair arithmetic does not depend on the grouping, so results equal the single-GPU engine's bit for
// bit, whatever the world size. NCCL is loaded at run time (the copy already in the process, if any).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include <cuda_runtime.h>

namespace rb200 {

// What one rank sends, receives and computes in one MoE layer, derived from all ranks' offsets.
struct EpPlan {
    std::vector<int32_t> send_begin, send_count;     // per peer: range of this rank's expert-sorted pairs
    std::vector<int32_t> recv_begin, recv_count;     // per peer: rows of the receive buffer
    std::vector<int32_t> offsets;                    // [n_expert + 1] over the receive buffer, non-local experts empty
    std::vector<int32_t> sorted;                     // receive-buffer rows grouped by expert (source rank order inside)
    int32_t n_recv = 0;
};

// all_offsets: [world][n_expert + 1] pair offsets of every rank (pairs sorted by expert id).
// n_expert must be a multiple of world. Pure host arithmetic.
void ep_make_plan(const int32_t * all_offsets, int world, int rank, int n_expert, EpPlan & plan);

// The NCCL entry points this path uses, resolved with dlopen / dlsym on first use.
struct NcclId128 { char bytes[128]; };       // ncclUniqueId, passed by value
struct NcclApi {
    void * lib = nullptr;
    int (*GetUniqueId)(void * id) = nullptr;
    int (*CommInitRank)(void ** comm, int nranks, NcclId128 id, int rank) = nullptr;
    int (*CommDestroy)(void * comm) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*Send)(const void * buf, size_t count, int dtype, int peer, void * comm, cudaStream_t stream) = nullptr;
    int (*Recv)(void * buf, size_t count, int dtype, int peer, void * comm, cudaStream_t stream) = nullptr;
    int (*AllGather)(const void * send, void * recv, size_t count, int dtype, void * comm, cudaStream_t stream) = nullptr;
    const char * (*GetErrorString)(int) = nullptr;
};
constexpr int kNcclInt32 = 2, kNcclFloat32 = 7;      // ncclInt32, ncclFloat32

// Throws std::runtime_error when the library or a symbol is missing.
const NcclApi & nccl_api();

// out[i][0..d) = x[sorted[i] / x_div][0..d)
void launch_ep_gather_rows(const float * x, int ldx, const int32_t * sorted, int x_div, int n, int d, float * out, cudaStream_t stream);
// out[sorted[i]][0..d) = in[i][0..d)
void launch_ep_scatter_rows(const float * in, const int32_t * sorted, int n, int d, float * out, int ldo, cudaStream_t stream);

} // namespace rb200
