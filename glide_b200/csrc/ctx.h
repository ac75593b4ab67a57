// The context behind the C ABI's opaque glide_ctx: one device, one stream, one scratch arena,
// and (optionally) one NCCL communicator for the calls that exchange rows between GPUs.
#pragma once

#include <cstdint>
#include <string>

#include <cuda_runtime.h>

struct glide_comm_state;   // comm.cu

struct glide_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr, ev_mid = nullptr;
    float split_ms[2] = {0.0f, 0.0f};  // last glide_search: routing pre-pass, search kernel
    std::string error;
    float last_ms = 0.0f;
    void *ws = nullptr;  // scratch, grown on demand
    size_t ws_bytes = 0;
    unsigned long long *counters = nullptr;  // 4 x u64 on the device
    uint32_t *ticket = nullptr;              // one word: the search kernel's query counter
    uint32_t *start_point_word = nullptr;    // one word: the start point of a per-partition refine
    uint32_t last_launches = 0;              // kernels enqueued by the last glide_search
    float *tc_norms = nullptr;               // centroid norms for the assignment's tensor-core prefilter (up to 4096 centroids)
    uint32_t tc_knn_fallbacks = 0;           // kNN stages the tensor-core kernel handed back to the fp32 kernels
    bool counters_on = false;
    glide_comm_state *comm = nullptr;        // NCCL communicator (glide_comm_init), or nullptr
};

// comm.cu: releases the communicator of a context that is being destroyed
void glide_comm_release(glide_ctx *ctx);
