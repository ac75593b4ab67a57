// Internal launcher interface between the C-ABI layer (api.cu) and the kernel
// translation units. Every launcher enqueues on `stream`, returns cudaError_t from
// the launch (no synchronisation) and never allocates.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace glide {

struct BeamParamsHost {
    uint32_t beam, max_iterations, min_iterations, hash_bit, hash_reset_interval;
};

// ---- search.cu -----------------------------------------------------------
// One partition of the large path as the device sees it (local ids; map: local id -> original id).
struct PartitionRef {
    const float *data;       // rows x dim; nullptr: the partition is not in device memory
    const uint32_t *graph;   // rows x degree
    const uint32_t *map;
    uint32_t start_point, rows;
};

struct SearchArgs {
    const float *data;           // n x dim
    const uint32_t *graph;       // n x degree
    uint32_t degree, dim;
    const float *queries;        // Q x dim
    uint32_t Q, top_k;
    int metric;
    BeamParamsHost p;
    // routed (small path): nearest centroid -> start point
    const float *centroids;      // C x dim
    uint32_t C;
    const uint32_t *route;       // Q: nearest centroid of every query (launch_assign)
    const uint32_t *start_points;
    uint32_t *out_ids;           // Q x top_k
    float *out_dists;            // Q x top_k
    // per-partition (large path): only queries routed to segment_id run
    const uint32_t *segment_ids; // Q x segment_num, or nullptr for the small path
    uint32_t segment_num, segment_id, start_point;
    const uint32_t *map;         // local id -> global id (large path)
    const PartitionRef *parts;   // large path, every partition in device memory: a query walks ALL the partitions it is
                                 // routed to inside one launch, in ascending partition order (segment_id is then unused)
    unsigned long long *counters;  // [0] data rows read, [1] expansions; may be nullptr
    const uint32_t *order;       // ticket t is query order[t] (queries grouped by partition: warps that run together
                                 // share L2 lines); nullptr: query t
    uint32_t *ticket;            // one word, zeroed by launch_search: warps draw their next query from it;
                                 // nullptr: query q runs on warp q of the grid
};
cudaError_t launch_search(const SearchArgs &a, cudaStream_t stream);
cudaError_t preload_search_kernels(cudaStream_t stream);

struct SelectSegmentArgs {
    const float *queries;
    uint32_t Q, dim;
    const float *centroids;
    uint32_t C, min_segment_num;
    float boundary_factor;
    int metric;
    uint32_t *out;  // Q x C
};
cudaError_t launch_select_segments(const SelectSegmentArgs &a, cudaStream_t stream);

// ---- graph_build.cu ------------------------------------------------------
enum BuildMode : int { kModeBuild = 0, kModeBoundary = 1, kModeRefine = 2, kModeRefineRow = 3 };

struct BuildArgs {
    int mode;
    const float *data;
    uint32_t dim;
    const uint32_t *graph_in;  // kNN graph (build/boundary) or the merged graph snapshot (refine)
    uint32_t in_degree;
    uint32_t *graph_out;
    uint32_t out_first;        // refine (and build with rows_by_point): row of point p is written at graph_out + (p - out_first) * out_degree
    int rows_by_point;         // build: rows are written by reorder position (see out_first) instead of by original id
    uint32_t out_degree;
    const uint32_t *seg_start, *seg_len;  // device, S entries (build/boundary)
    uint32_t S;
    const uint32_t *start_points;  // build: partition-local per segment; refine: per centroid, graph ids
    const uint32_t *map;           // reorder id -> original id; nullptr = identity
    const float *centroids;        // refine
    uint32_t C;
    const uint32_t *route;         // refine: nearest centroid of points route_first, route_first+1, ... (launch_assign)
    uint32_t route_first;
    const uint32_t *order;         // refine: warp t handles point first + order[t] (points grouped by partition so that
                                   // warps running together share L2 lines); nullptr: first + t
    uint32_t first, count;         // point range handled by this launch
    const uint32_t *count_dev;     // when set: the number of entries of `order` to handle, read on the device (the
                                   // grid still covers `count`; warps beyond *count_dev leave at once)
    uint32_t fixed_segment;        // boundary: the segment every point belongs to
    uint32_t max_seg_rows;         // build/boundary: rows of the largest partition this launch can touch (0: not known);
                                   // lets the launcher take the bitmap form of the visited set
    float alpha;
    int metric;
    BeamParamsHost p;
    unsigned long long *counters;  // [0] rows read in search, [1] expansions, [2] rows read in pruning
};
cudaError_t launch_build(const BuildArgs &a, cudaStream_t stream);
cudaError_t preload_build_kernels(cudaStream_t stream);
// The rows of graph[first .. first + count) that hold at least one empty slot, as indices relative to
// `first`, in the order of order_in (nullptr: ascending); *count_out receives how many. flags: count
// words of scratch. A refine launch over that list keeps every warp of a CTA busy; one over all rows
// leaves most CTAs with a warp or two at work when few rows have holes.
cudaError_t launch_rows_with_holes(const uint32_t *graph, uint32_t first, uint32_t count, uint32_t degree,
                                   const uint32_t *order_in, uint32_t *flags, uint32_t *order_out, uint32_t *count_out,
                                   cudaStream_t stream);

struct ReverseArgs {
    uint32_t *graph;   // num x degree, updated in place
    uint32_t num, degree;
    // scratch: counts[num+1], offsets[num+1] u32; edges: u64 [num*degree]
    uint32_t *counts;
    uint32_t *offsets;
    unsigned long long *edges;
    void *scan_tmp;       // >= reverse_scan_tmp_bytes(num)
};
size_t reverse_scan_tmp_bytes(uint32_t num);
cudaError_t launch_reverse(const ReverseArgs &a, cudaStream_t stream);

// ---- partition.cu --------------------------------------------------------
cudaError_t launch_gather_rows(const float *data, const uint32_t *ids, uint32_t count, uint32_t dim, float *out,
                               cudaStream_t stream);
struct AssignArgs {
    const float *data;
    uint32_t n, dim;
    const float *centroids;
    uint32_t C;
    float boundary_factor;  // < 0: no boundary test (large path, k-means)
    int metric;
    uint32_t *nearest;      // n
    uint32_t *is_boundary;  // n: 0 for a boundary point, 0xffffffff otherwise (a slot key); may be nullptr
    float *tc_norms;        // scratch for the tensor-core prefilter: C rounded up to a multiple of 128, plus 1,
                            // floats (norms, padding, their maximum at [C]); nullptr: exact kernels only
    unsigned long long *fallback_counter;  // += points settled by the warp-per-point kernel; may be nullptr
};
// *launched (optional) receives the number of kernels this call enqueued
cudaError_t launch_assign(const AssignArgs &a, cudaStream_t stream, uint32_t *launched = nullptr);
// Tensor-core prefilter + exact re-rank (assign_tc.cu); settles every point whose nearest centroid
// is unique, flags the rest with 0xffffffff in `nearest`. Eligible: tc_norms given, dim % 16 == 0, dim <= 128, C >= 2.
bool assign_tc_eligible(const AssignArgs &a);
cudaError_t launch_assign_tc(const AssignArgs &a, cudaStream_t stream);   // two kernels: norms, prefilter + re-rank

// Deterministic slots: slot[p] = number of q < p with key[q] == key[p] (keys < K,
// key == 0xffffffff means "none" and yields slot 0xffffffff); totals[K] = counts.
// scratch: block_hist words = slot_scratch_words(n, K).
// order[] = 0..n-1 grouped by key (keys < K <= 4096; every key must be valid), one CTA; for small n.
cudaError_t launch_group_by_key(const uint32_t *key, uint32_t n, uint32_t K, uint32_t *order, cudaStream_t stream);
size_t slot_scratch_words(uint32_t n, uint32_t K);
cudaError_t launch_slots(const uint32_t *key, uint32_t n, uint32_t K, uint32_t *slot, uint32_t *totals,
                         uint32_t *scratch, cudaStream_t stream);
cudaError_t launch_reorder(const float *data, uint32_t n, uint32_t dim, const uint32_t *seg_index,
                           const uint32_t *seg_start_dev, float *reorder_data, uint32_t *map, cudaStream_t stream);
cudaError_t launch_pack_seg_index(const uint32_t *nearest, const uint32_t *slot, const uint32_t *bslot, uint32_t n,
                                  uint32_t *seg_index, cudaStream_t stream);
// k-means centroid update: members of cluster c are member_ids[off[c] .. off[c]+cnt[c]) in ascending row order.
cudaError_t launch_centroid_update(const float *sample, uint32_t dim, const uint32_t *member_ids,
                                   const uint32_t *off, const uint32_t *cnt, uint32_t C, float *centroids,
                                   cudaStream_t stream);
cudaError_t launch_scatter_members(const uint32_t *label, const uint32_t *slot, const uint32_t *off, uint32_t n,
                                   uint32_t *member_ids, cudaStream_t stream);
// k-means initialisation by farthest-first traversal of the sample rows.
size_t farthest_first_scratch_bytes(uint32_t n);
cudaError_t launch_farthest_first(const float *sample, uint32_t n, uint32_t dim, uint32_t C, float *centroids,
                                  void *scratch, cudaStream_t stream);
cudaError_t launch_count_changed(const uint32_t *a, const uint32_t *b, uint32_t n, uint32_t *count,
                                 cudaStream_t stream);

// ---- bruteforce.cu -------------------------------------------------------
size_t bruteforce_scratch_bytes(uint32_t Q, uint32_t k, uint32_t splits);
uint32_t bruteforce_default_splits(uint32_t n, uint32_t Q);
cudaError_t launch_bruteforce(const float *base, uint32_t n, const float *queries, uint32_t Q, uint32_t dim,
                              uint32_t k, int metric, uint32_t splits, void *scratch, uint32_t *out_ids,
                              float *out_dists, cudaStream_t stream);

// Exact kNN graph of every partition of at most max_len rows (all pairs inside the
// partition). Tiles: 3 words each (segment start, segment length, first row), built on the host.
uint32_t segment_knn_tile_count(const uint32_t *h_seg_len, uint32_t S, uint32_t max_len);
void segment_knn_fill_tiles(const uint32_t *h_seg_start, const uint32_t *h_seg_len, uint32_t S, uint32_t max_len,
                            uint32_t *h_tiles);
// row_base: index of data's row 0 within the whole reordered set (enters the padding hash of short partitions)
cudaError_t launch_segment_knn(const float *data, uint32_t dim, const uint32_t *d_tiles, uint32_t tile_count,
                               uint32_t out_degree, uint32_t row_base, int32_t *out, cudaStream_t stream);

// ---- knn_tc.cu -----------------------------------------------------------
// Exact per-partition kNN rows on the tensor cores (TF32 Gram tiles by TMA + tcgen05, threshold
// selection, exact fp32 re-rank). Eligible: dim a multiple of 32 up to 128, out_degree <= 64, rows
// 16-byte aligned, tensor maps available.
bool knn_tc_eligible(const float *data, uint32_t dim, uint32_t out_degree);
size_t knn_tc_scratch_bytes(uint64_t rows_total, uint32_t out_degree);
// Partitions s with 1 <= h_seg_len[s] <= max_len (rows [h_seg_start[s], +len) of data). Synchronises the
// stream. *h_failed != 0: a bounded wait ran out, recompute the rows with another kernel.
cudaError_t launch_knn_tc(const float *data, uint64_t rows_total, uint32_t dim, const uint32_t *h_seg_start,
                          const uint32_t *h_seg_len, uint32_t S, uint32_t max_len, uint32_t out_degree, uint32_t row_base,
                          void *scratch, int32_t *out, uint32_t *h_failed, cudaStream_t stream);

// ---- nn_descent.cu -------------------------------------------------------
struct NndArgs {
    const float *data;   // rows x dim (reorder space)
    uint32_t rows, dim;
    const uint32_t *seg_start, *seg_len;  // device, S entries
    uint32_t S;
    uint32_t min_seg_len;  // partitions with fewer rows are skipped (handled by the exact all-pairs kernel)
    uint32_t K;          // list width (multiple of 32, <= 64)
    uint32_t sample;     // new/old samples per direction (<= 32)
    uint32_t max_iterations;
    float termination_threshold;
    uint64_t seed;
    int metric;
    // state (device): lists keys u64 [rows*K]; proposal slots u64 [rows*P]; samples
    void *workspace;
    size_t workspace_bytes;
    int32_t *out_knn;    // rows x out_degree, partition-local ids
    uint32_t out_degree;
    uint32_t row_base;         // index of row 0 within the whole reordered set (seeds and padding hash global row numbers,
                               // so a sharded run gives the rows of the whole run)
    uint32_t *iterations_run;  // host pointer, may be nullptr
    float *stage_ms;           // host pointer [3] (sample, join, merge), may be nullptr
};
size_t nnd_workspace_bytes(uint32_t rows, uint32_t K, uint32_t sample, uint32_t S);
cudaError_t run_nn_descent(const NndArgs &a, cudaStream_t stream);

// ---- large.cu -------------------------------------------------------------
// count uint8 values -> fp32 (count % 4 == 0)
cudaError_t launch_widen_u8(const uint8_t *in, float *out, size_t count, cudaStream_t stream);

}  // namespace glide
