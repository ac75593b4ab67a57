// Harness around the REFERENCE's own kernels, used only to pin the CPU oracle.
//
// TEST INFRASTRUCTURE. This file contains no reference code: it includes the reference's
// RAFT-free kernel headers from where they lie (-I<reference>/src: search_kernel.cuh,
// graph_kernel.cuh, partition_kernel.cuh and what they include) and launches them the way the
// reference's host code does, citing the lines it mirrors. It is compiled by oracle/Makefile into
// oracle/_ref/libglide_ref.so only when the reference tree is present; the binary is never
// committed. params.cuh names three raft::host_vector_view members (params.cuh:32-34); the
// stand-in below gives that name a body so the header compiles without RAFT.
#include <cstdint>
#include <cstdio>
#include <climits>
#include <cfloat>
#include <algorithm>
#include <cuda_runtime.h>

namespace raft {
template<typename T>
struct host_vector_view {
    T *ptr = nullptr;
    size_t n = 0;
};
}  // namespace raft

#include "graph_kernel.cuh"      // includes search_kernel.cuh, distance.cuh, bitonic.cuh, hashmap.cuh, utils.cuh, params.cuh
#include "partition_kernel.cuh"

namespace {

inline uint32_t round_up32(uint32_t x) { return (x + 31u) & ~31u; }

#define REF_CHECK(call)                                                                 \
    do {                                                                                \
        cudaError_t e_ = (call);                                                        \
        if (e_ != cudaSuccess) {                                                        \
            std::fprintf(stderr, "ref_harness: %s: %s\n", #call, cudaGetErrorString(e_)); \
            return -3;                                                                  \
        }                                                                               \
    } while (0)

// Device time of the kernels of the last call, taken with events on the default stream.
float g_last_ms = 0.0f;
struct EventTimer {
    cudaEvent_t a = nullptr, b = nullptr;
    EventTimer() { cudaEventCreate(&a); cudaEventCreate(&b); cudaEventRecord(a, 0); }
    void stop() { cudaEventRecord(b, 0); cudaEventSynchronize(b); cudaEventElapsedTime(&g_last_ms, a, b); }
    ~EventTimer() { cudaEventDestroy(a); cudaEventDestroy(b); }
};

// the beam ladder of kernel_config.cuh:40-48 for MAX_CANDIDATE = 64
template<typename F64, typename F128, typename F256>
int by_beam(uint32_t beam, F64 f64, F128 f128, F256 f256) {
    if (beam <= 64) return f64();
    if (beam <= 128) return f128();
    if (beam <= 256) return f256();
    return -2;
}

}  // namespace

extern "C" {

float ref_last_ms() { return g_last_ms; }

// GLIDE::search launch, glide_impl.cuh:389-437, block size 64 (kernel_config.cuh:11). MAX_CENTROID is 32 up
// to 32 centroids and, for adjacency rows of at most 64 entries, 64 beyond (kernel_config.cuh:206-216:
// the reference takes it from graph_degree there, so more than 64 centroids would be silently cut).
int ref_search(const float *d_data, uint32_t dim, const uint32_t *d_graph, uint32_t degree, const float *d_centroids,
               uint32_t C, const uint32_t *d_start_points, const float *d_queries, uint32_t Q, uint32_t top_k,
               uint32_t beam, uint32_t max_iterations, uint32_t min_iterations, uint32_t hash_bit,
               uint32_t hash_reset_interval, int metric, uint32_t *d_ids, float *d_dists) {
    if (degree > 256 || beam > 512 || C > 64 || (C > 32 && (degree > 64 || beam > 256))) return -2;
    const uint32_t rbs = round_up32(beam + degree);
    if (C > rbs) return -2;  // the centroid lists alias the result buffers (search_kernel.cuh:424-427)
    const uint32_t smem = dim * sizeof(float) + rbs * (sizeof(uint32_t) + sizeof(float)) +
                          hashmap::get_size(hash_bit) * sizeof(uint32_t) + 5 * sizeof(uint32_t);
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -3;
        kernel<<<Q, 64, smem>>>(d_ids, d_dists, top_k, d_data, d_queries, d_graph, degree, beam, max_iterations,
                                min_iterations, hash_bit, hash_reset_interval, d_start_points, dim, C, d_centroids, m);
        return 0;
    };
    int rc;
    if (C <= 32 && (degree > 64 || beam > 256)) {
        // the wider ladders (kernel_config.cuh:40-60): MAX_CANDIDATE 128 / 256 and MAX_BEAM 512, the sizes at
        // which the reference sorts and merges with two warps (search_kernel.cuh:38-95, 148-233)
        auto by_beam4 = [&](auto k64, auto k128, auto k256, auto k512) {
            if (beam <= 64) return launch(k64);
            if (beam <= 128) return launch(k128);
            if (beam <= 256) return launch(k256);
            return launch(k512);
        };
        if (degree <= 64)
            rc = by_beam4(search_kernel<64, 64, 32, float, uint32_t>, search_kernel<64, 128, 32, float, uint32_t>,
                          search_kernel<64, 256, 32, float, uint32_t>, search_kernel<64, 512, 32, float, uint32_t>);
        else if (degree <= 128)
            rc = by_beam4(search_kernel<128, 64, 32, float, uint32_t>, search_kernel<128, 128, 32, float, uint32_t>,
                          search_kernel<128, 256, 32, float, uint32_t>, search_kernel<128, 512, 32, float, uint32_t>);
        else
            rc = by_beam4(search_kernel<256, 64, 32, float, uint32_t>, search_kernel<256, 128, 32, float, uint32_t>,
                          search_kernel<256, 256, 32, float, uint32_t>, search_kernel<256, 512, 32, float, uint32_t>);
    } else if (C <= 32)
        rc = by_beam(beam, [&] { return launch(search_kernel<64, 64, 32, float, uint32_t>); },
                     [&] { return launch(search_kernel<64, 128, 32, float, uint32_t>); },
                     [&] { return launch(search_kernel<64, 256, 32, float, uint32_t>); });
    else
        rc = by_beam(beam, [&] { return launch(search_kernel<64, 64, 64, float, uint32_t>); },
                     [&] { return launch(search_kernel<64, 128, 64, float, uint32_t>); },
                     [&] { return launch(search_kernel<64, 256, 64, float, uint32_t>); });
    if (rc) return rc;
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// GLIDE::subgraph_build_and_merge launches, glide_impl.cuh:99-187.
int ref_build(const float *d_reorder, uint32_t reorder_num, uint32_t dim, const uint32_t *d_knn, uint32_t knn_degree,
              const uint32_t *d_seg_start, const uint32_t *d_seg_len, uint32_t segment_num,
              const uint32_t *d_start_points_local, const uint32_t *d_map, uint32_t num, uint32_t graph_degree,
              uint32_t beam, uint32_t max_iterations, uint32_t min_iterations, uint32_t hash_bit,
              uint32_t hash_reset_interval, float relaxant_factor, int metric, int with_boundary, uint32_t *d_graph) {
    if (knn_degree > 64) return -2;
    const uint32_t rbs = round_up32(beam + knn_degree);
    const uint32_t bitmap_size = (beam + 31) / 32;
    const uint32_t max_graph_degree = round_up32(graph_degree);
    uint32_t smem = dim * sizeof(float) + rbs * (sizeof(uint32_t) + sizeof(float)) + max_graph_degree * sizeof(uint32_t) +
                    hashmap::get_size(hash_bit) * sizeof(uint32_t) + 7 * sizeof(uint32_t) + bitmap_size * sizeof(uint32_t);
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch1 = [&](auto kernel) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -3;
        kernel<<<num, 64, smem>>>(d_reorder, d_graph, d_start_points_local, d_seg_start, d_seg_len, knn_degree, graph_degree,
                                  max_graph_degree, segment_num, dim, d_map, d_knn, beam, hash_bit, hash_reset_interval,
                                  max_iterations, min_iterations, num, 0u, relaxant_factor, m);
        return 0;
    };
    int rc = by_beam(beam, [&] { return launch1(build_kernel<64, 64, float, uint32_t>); },
                     [&] { return launch1(build_kernel<64, 128, float, uint32_t>); },
                     [&] { return launch1(build_kernel<64, 256, float, uint32_t>); });
    if (rc) return rc;
    REF_CHECK(cudaGetLastError());
    REF_CHECK(cudaDeviceSynchronize());
    const uint32_t boundary_num = reorder_num - num;
    if (with_boundary && boundary_num > 0) {
        smem += max_graph_degree * sizeof(uint32_t);
        auto launch2 = [&](auto kernel) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -3;
            kernel<<<boundary_num, 64, smem>>>(d_reorder, d_graph, d_start_points_local, knn_degree, graph_degree,
                                               max_graph_degree, dim, bitmap_size, segment_num - 1, num, d_map, d_knn, beam,
                                               hash_bit, hash_reset_interval, max_iterations, min_iterations, reorder_num, num,
                                               relaxant_factor, m);
            return 0;
        };
        rc = by_beam(beam, [&] { return launch2(build_boundary_kernel<64, 64, float, uint32_t>); },
                     [&] { return launch2(build_boundary_kernel<64, 128, float, uint32_t>); },
                     [&] { return launch2(build_boundary_kernel<64, 256, float, uint32_t>); });
        if (rc) return rc;
        REF_CHECK(cudaGetLastError());
        REF_CHECK(cudaDeviceSynchronize());
    }
    timer.stop();
    return 0;
}

// GLIDE::reverse_graph, glide_impl.cuh:194-256, with the `degree` launches issued one after
// another on one stream (the reference spreads them over pool streams).
int ref_reverse(uint32_t *d_graph, uint32_t num, uint32_t degree) {
    uint32_t *rev = nullptr, *cnt = nullptr, *dst = nullptr;
    REF_CHECK(cudaMalloc(&rev, (size_t) num * degree * 4));
    REF_CHECK(cudaMalloc(&cnt, (size_t) num * 4));
    REF_CHECK(cudaMalloc(&dst, (size_t) num * 4));
    REF_CHECK(cudaMemset(rev, 0xff, (size_t) num * degree * 4));
    REF_CHECK(cudaMemset(cnt, 0, (size_t) num * 4));
    EventTimer timer;
    for (uint32_t k = 0; k < degree; k++)
        reverse_graph_kernel<uint32_t><<<(num + 511) / 512, 512>>>(dst, rev, cnt, d_graph, num, degree, k);
    const uint32_t max_graph_degree = round_up32(degree);
    insert_reverse_kernel<uint32_t><<<num, 32, max_graph_degree * 4>>>(d_graph, rev, cnt, num, degree, max_graph_degree);
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    cudaFree(rev); cudaFree(cnt); cudaFree(dst);
    return 0;
}

// GLIDE::refine launch, glide_impl.cuh:270-312. In place, as the reference does.
int ref_refine(const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph, uint32_t degree,
               const float *d_centroids, uint32_t C, const uint32_t *d_start_points, uint32_t beam,
               uint32_t max_iterations, uint32_t min_iterations, uint32_t hash_bit, uint32_t hash_reset_interval,
               float relaxant_factor, int metric) {
    if (degree > 64 || C > 64) return -2;
    const uint32_t rbs = round_up32(beam + degree);
    if (C > rbs) return -2;  // the centroid lists alias the result buffers
    const uint32_t bitmap_size = (beam + 31) / 32;
    const uint32_t max_graph_degree = round_up32(degree);
    const uint32_t smem = dim * sizeof(float) + rbs * (sizeof(uint32_t) + sizeof(float)) + 2 * max_graph_degree * sizeof(uint32_t) +
                          hashmap::get_size(hash_bit) * sizeof(uint32_t) + 9 * sizeof(uint32_t) + bitmap_size * sizeof(uint32_t);
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -3;
        kernel<<<num, 64, smem>>>(d_data, d_graph, d_start_points, d_centroids, degree, max_graph_degree, dim, beam, hash_bit,
                                  hash_reset_interval, max_iterations, min_iterations, num, C, relaxant_factor, 0u, m);
        return 0;
    };
    int rc;
    if (C <= 32)   // kernel_config.cuh:161-171
        rc = by_beam(beam, [&] { return launch(refine_kernel<64, 64, 32, float, uint32_t>); },
                     [&] { return launch(refine_kernel<64, 128, 32, float, uint32_t>); },
                     [&] { return launch(refine_kernel<64, 256, 32, float, uint32_t>); });
    else
        rc = by_beam(beam, [&] { return launch(refine_kernel<64, 64, 64, float, uint32_t>); },
                     [&] { return launch(refine_kernel<64, 128, 64, float, uint32_t>); },
                     [&] { return launch(refine_kernel<64, 256, 64, float, uint32_t>); });
    if (rc) return rc;
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// define_partition launch, partition.cuh:79-100 (256 threads; MAX_CENTROID ladder kernel_config.cuh:218-235).
int ref_define_partition(const float *d_data, uint32_t num, uint32_t dim, float *d_centroids, uint32_t C,
                         float boundary_factor, int metric, uint32_t *d_segment_lengths, uint32_t *d_segment_indexes) {
    if (C > 256) return -2;
    REF_CHECK(cudaMemset(d_segment_lengths, 0, (size_t) (C + 1) * 4));
    const uint32_t smem = dim * sizeof(float) + C * (sizeof(float) + sizeof(uint32_t));
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        kernel<<<num, 256, smem>>>(d_data, d_centroids, num, dim, C, d_segment_lengths, d_segment_indexes, boundary_factor, m);
    };
    if (C <= 32) launch(define_partition_kernel<32, float, uint32_t>);
    else if (C <= 64) launch(define_partition_kernel<64, float, uint32_t>);
    else if (C <= 128) launch(define_partition_kernel<128, float, uint32_t>);
    else launch(define_partition_kernel<256, float, uint32_t>);
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// reorder launch, partition.cuh:135-151 (128 threads, one block per point).
int ref_reorder(const float *d_data, float *d_reorder, const uint32_t *d_segment_indexes, uint32_t *d_map,
                const uint32_t *d_segment_starts, uint32_t num, uint32_t dim) {
    EventTimer timer;
    reorder_kernel<float, uint32_t><<<num, 128>>>(d_data, d_reorder, d_segment_indexes, d_map, d_segment_starts, num, dim);
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// ---- large path. The reference's large-path classes are instantiated for uint8 rows
// (large_build.cu:84, large_search.cu) and search_on_sub_kernel keeps its query in a uint8 buffer
// whatever Data_t is (search_kernel.cuh:666), so the harness runs these kernels on uint8 rows;
// integer-valued rows make every distance exact, so the oracle on the same values as fp32 must
// agree bit for bit. ----

// define_partition_for_large launch, partition.cuh:290-318 (128 threads; no boundary test).
int ref_define_partition_for_large(const uint8_t *d_data, uint32_t batch_size, uint32_t dim, float *d_centroids, uint32_t C,
                                   int metric, uint32_t *d_segment_lengths, uint32_t *d_segment_indexes) {
    if (C > 256 || dim % 4) return -2;
    REF_CHECK(cudaMemset(d_segment_lengths, 0, (size_t) C * 4));
    const uint32_t smem = dim * sizeof(uint8_t) + C * (sizeof(float) + sizeof(uint32_t));
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        kernel<<<batch_size, 128, smem>>>(d_data, d_centroids, batch_size, dim, C, d_segment_lengths, d_segment_indexes, m);
    };
    if (C <= 32) launch(define_partition_for_large_kernel<32, uint8_t, uint32_t>);
    else if (C <= 64) launch(define_partition_for_large_kernel<64, uint8_t, uint32_t>);
    else if (C <= 128) launch(define_partition_for_large_kernel<128, uint8_t, uint32_t>);
    else launch(define_partition_for_large_kernel<256, uint8_t, uint32_t>);
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// GLIDE_large::subgraph_build launch for one resident partition, glide_large_impl.cuh:95-157.
int ref_build_for_large(const uint8_t *d_data, uint32_t length, uint32_t dim, const uint32_t *d_knn, uint32_t knn_degree,
                        uint32_t start_point, uint32_t graph_degree, uint32_t beam, uint32_t max_iterations,
                        uint32_t min_iterations, uint32_t hash_bit, uint32_t hash_reset_interval, float relaxant_factor,
                        int metric, uint32_t *d_graph) {
    if (knn_degree > 64 || dim % 4) return -2;
    const uint32_t rbs = round_up32(beam + knn_degree);
    const uint32_t bitmap_size = (beam + 31) / 32;
    const uint32_t max_graph_degree = round_up32(graph_degree);
    const uint32_t smem = dim * sizeof(uint8_t) + rbs * (sizeof(uint32_t) + sizeof(float)) + max_graph_degree * sizeof(uint32_t) +
                          hashmap::get_size(hash_bit) * sizeof(uint32_t) + 7 * sizeof(uint32_t) + bitmap_size * sizeof(uint32_t);
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -3;
        kernel<<<length, 64, smem>>>(d_data, d_graph, start_point, knn_degree, graph_degree, max_graph_degree, dim, d_knn, beam,
                                     hash_bit, hash_reset_interval, max_iterations, min_iterations, length, 0u,
                                     relaxant_factor, m);
        return 0;
    };
    int rc = by_beam(beam, [&] { return launch(build_for_large_kernel<64, 64, uint8_t, uint32_t>); },
                     [&] { return launch(build_for_large_kernel<64, 128, uint8_t, uint32_t>); },
                     [&] { return launch(build_for_large_kernel<64, 256, uint8_t, uint32_t>); });
    if (rc) return rc;
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// GLIDE_large::refine launch for one resident partition, glide_large_impl.cuh:257-318. In place.
int ref_refine_for_large(const uint8_t *d_data, uint32_t length, uint32_t dim, uint32_t *d_graph, uint32_t graph_degree,
                         uint32_t start_point, uint32_t beam, uint32_t max_iterations, uint32_t min_iterations,
                         uint32_t hash_bit, uint32_t hash_reset_interval, float relaxant_factor, int metric) {
    if (graph_degree > 64 || dim % 4) return -2;
    const uint32_t rbs = round_up32(beam + graph_degree);
    const uint32_t bitmap_size = (beam + 31) / 32;
    const uint32_t max_graph_degree = round_up32(graph_degree);
    const uint32_t smem = dim * sizeof(uint8_t) + rbs * (sizeof(uint32_t) + sizeof(float)) + 2 * max_graph_degree * sizeof(uint32_t) +
                          hashmap::get_size(hash_bit) * sizeof(uint32_t) + 9 * sizeof(uint32_t) + bitmap_size * sizeof(uint32_t);
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -3;
        kernel<<<length, 64, smem>>>(d_data, d_graph, start_point, graph_degree, max_graph_degree, dim, beam, hash_bit,
                                     hash_reset_interval, max_iterations, min_iterations, length, relaxant_factor, 0u, m);
        return 0;
    };
    int rc = by_beam(beam, [&] { return launch(refine_for_large_kernel<64, 64, uint8_t, uint32_t>); },
                     [&] { return launch(refine_for_large_kernel<64, 128, uint8_t, uint32_t>); },
                     [&] { return launch(refine_for_large_kernel<64, 256, uint8_t, uint32_t>); });
    if (rc) return rc;
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// GLIDE_large::search, routing step, glide_large_impl.cuh:385-416 (128 threads). The reference never
// initialises the Q x C output (only the kernel's first C words, search_kernel.cuh:563-565); the
// harness fills it with 0xffffffff first, which is what the consumer's loop expects
// (search_kernel.cuh:683-688).
int ref_select_segments(const uint8_t *d_queries, uint32_t Q, uint32_t dim, const float *d_centroids, uint32_t C,
                        uint32_t min_segment_num, float boundary_factor, int metric, uint32_t *d_segment_ids) {
    if (C > 256 || dim % 4) return -2;
    REF_CHECK(cudaMemset(d_segment_ids, 0xff, (size_t) Q * C * 4));
    const uint32_t smem = dim * sizeof(uint8_t) + C * (sizeof(uint32_t) + sizeof(float));
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        kernel<<<Q, 128, smem>>>(d_segment_ids, d_queries, d_centroids, C, dim, min_segment_num, boundary_factor, m);
    };
    if (C <= 32) launch(select_segment_kernel<32, uint8_t, uint32_t>);
    else if (C <= 64) launch(select_segment_kernel<64, uint8_t, uint32_t>);
    else if (C <= 128) launch(select_segment_kernel<128, uint8_t, uint32_t>);
    else launch(select_segment_kernel<256, uint8_t, uint32_t>);
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

// GLIDE_large::search, one resident partition, glide_large_impl.cuh:440-488 (64 threads; MAX_TOPK
// ladder kernel_config.cuh:309-319).
int ref_search_on_sub(const uint8_t *d_data, uint32_t dim, const uint32_t *d_graph, uint32_t graph_degree, uint32_t *d_map,
                      uint32_t start_point, const uint8_t *d_queries, uint32_t Q, const uint32_t *d_segment_ids,
                      uint32_t segment_num, uint32_t segment_id, uint32_t top_k, uint32_t beam, uint32_t max_iterations,
                      uint32_t min_iterations, uint32_t hash_bit, uint32_t hash_reset_interval, int metric,
                      uint32_t *d_final_ids, float *d_final_dists) {
    if (graph_degree > 64 || top_k > 128 || dim % 4) return -2;
    const uint32_t rbs = round_up32(beam + graph_degree);
    const uint32_t smem = dim * sizeof(uint8_t) + rbs * (sizeof(uint32_t) + sizeof(float)) +
                          hashmap::get_size(hash_bit) * sizeof(uint32_t) + 6 * sizeof(uint32_t);
    const Metric m = metric == 0 ? Metric::Euclidean : Metric::Cosine;
    EventTimer timer;
    auto launch = [&](auto kernel) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -3;
        kernel<<<Q, 64, smem>>>(d_final_ids, d_final_dists, top_k, d_data, d_queries, d_segment_ids, d_graph, d_map,
                                graph_degree, segment_num, segment_id, beam, max_iterations, min_iterations, hash_bit,
                                hash_reset_interval, start_point, dim, m);
        return 0;
    };
    int rc;
    if (top_k <= 32)
        rc = by_beam(beam, [&] { return launch(search_on_sub_kernel<64, 64, 32, uint8_t, uint32_t>); },
                     [&] { return launch(search_on_sub_kernel<64, 128, 32, uint8_t, uint32_t>); },
                     [&] { return launch(search_on_sub_kernel<64, 256, 32, uint8_t, uint32_t>); });
    else if (top_k <= 64)
        rc = by_beam(beam, [&] { return launch(search_on_sub_kernel<64, 64, 64, uint8_t, uint32_t>); },
                     [&] { return launch(search_on_sub_kernel<64, 128, 64, uint8_t, uint32_t>); },
                     [&] { return launch(search_on_sub_kernel<64, 256, 64, uint8_t, uint32_t>); });
    else
        rc = by_beam(beam, [&] { return launch(search_on_sub_kernel<64, 64, 128, uint8_t, uint32_t>); },
                     [&] { return launch(search_on_sub_kernel<64, 128, 128, uint8_t, uint32_t>); },
                     [&] { return launch(search_on_sub_kernel<64, 256, 128, uint8_t, uint32_t>); });
    if (rc) return rc;
    REF_CHECK(cudaGetLastError());
    timer.stop();
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

}  // extern "C"
