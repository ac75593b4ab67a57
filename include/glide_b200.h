/*
 * glide_b200 — C ABI of the B200-native GLIDE hot path.
 *
 * A drop-in for the stages of owlet-hub/GLIDE's pipeline: partition -> kNN graph ->
 * graph build/refine -> search (small, GPU-resident variant and large, per-partition
 * variant). Every entry point takes plain pointers and sizes; pointers named d_* are
 * device pointers, h_* host pointers. Matrices are row-major; ids are uint32_t; an
 * empty graph slot is 0xffffffff. All calls return 0 on success or a negative
 * glide_status; glide_last_error() gives the message of the last failure on a context.
 * Work is enqueued on the context's stream and the call returns after that stream has
 * been synchronised unless stated otherwise.
 *
 * Each declaration names the reference interface it replaces (paths relative to the
 * reference's src/ directory).
 */
#ifndef GLIDE_B200_H
#define GLIDE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct glide_ctx glide_ctx;

typedef enum {
    GLIDE_OK = 0,
    GLIDE_ERR_BAD_ARG = -1,      /* null pointer, zero size, inconsistent sizes */
    GLIDE_ERR_UNSUPPORTED = -2,  /* beam > 512, degree > 256, ... (kernel_config.cuh:47-48, :59-60) */
    GLIDE_ERR_CUDA = -3,         /* a CUDA call failed; see glide_last_error */
    GLIDE_ERR_NO_MEMORY = -4,
    GLIDE_ERR_IO = -5,
    GLIDE_ERR_NCCL = -6          /* libnccl could not be opened, or an NCCL call failed; see glide_last_error */
} glide_status;

enum { GLIDE_METRIC_EUCLIDEAN = 0, GLIDE_METRIC_COSINE = 1 }; /* params.cuh:5-8 */

/* SearchParameter, params.cuh:37-47, after adjust_search_params / calculate_hash_* (:49-99). */
typedef struct {
    uint32_t top_k;
    uint32_t beam;                /* multiple of 32, <= 512 */
    uint32_t max_iterations;      /* >= 1 */
    uint32_t min_iterations;
    uint32_t hash_bit;            /* 8..13 */
    uint32_t hash_reset_interval; /* >= 1 */
} glide_search_params;

/* ---- context ------------------------------------------------------------------------- */
/* The reference hard-codes cudaSetDevice(1) in every main (small_build.cu:33); here the
 * device is a parameter. Creates one stream. */
int glide_ctx_create(int device, glide_ctx **out);
void glide_ctx_destroy(glide_ctx *ctx);
const char *glide_last_error(const glide_ctx *ctx);
/* cudaStream_t of the context, for callers that enqueue their own work around the calls. */
void *glide_ctx_stream(glide_ctx *ctx);
/* Bytes of the context's scratch arena (grown on demand by the calls that need scratch, never
 * shrunk before glide_ctx_destroy). No counterpart in the reference (RMM pools its memory). */
size_t glide_ctx_workspace_bytes(const glide_ctx *ctx);
/* Elapsed device milliseconds of the kernels of the most recent call on this context
 * (the reference's timing convention: cudaEvent pairs around kernels, glide_impl.cuh:144-147). */
float glide_last_kernel_ms(const glide_ctx *ctx);

/* Parameter helpers: params.cuh:49-66, :68-80, :82-99. */
uint32_t glide_calculate_hash_bitlen(uint32_t beam, uint32_t graph_degree, float max_fill_rate, uint32_t min_bitlen);
uint32_t glide_calculate_hash_reset_interval(uint32_t beam, uint32_t graph_degree, float max_fill_rate,
                                             uint32_t hash_bitlen);
void glide_adjust_search_params(uint32_t min_iterations, uint32_t *max_iterations, uint32_t *beam);

/* ---- partition stage (partition.cuh) ---------------------------------------------------- */
/* get_centroids, partition.cuh:8-59: sample floor(n*sample_factor) rows (seeded) and fit
 * `centroid_num` centroids: farthest-first initialisation, then Lloyd iterations (the
 * reference calls cuVS kmeans::fit, whose arithmetic is not part of its tree).
 * d_centroids: centroid_num x dim. */
int glide_get_centroids(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, uint32_t centroid_num,
                        float sample_factor, uint64_t seed, uint32_t max_iter, int metric, float *d_centroids,
                        uint32_t *iterations_run);
/* The sample rows get_centroids draws: an arithmetic progression modulo n with a seeded
 * stride coprime to n (the reference shuffles all ids, partition.cuh:25-31). */
int glide_sample_ids(uint32_t n, uint32_t sample_num, uint64_t seed, uint32_t *h_out);
/* k-means on rows already selected (the fit itself), for callers that sample themselves.
 * init 0: the first centroid_num rows; init 1: farthest-first traversal of the rows (what
 * glide_get_centroids uses). Lloyd rounds stop after max_iter (0 -> 25) or when no label changes. */
int glide_kmeans_fit(glide_ctx *ctx, const float *d_sample, uint32_t n, uint32_t dim, uint32_t centroid_num,
                     uint32_t max_iter, int metric, int init, float *d_centroids, uint32_t *d_labels_or_null,
                     uint32_t *iterations_run);
/* define_partition, partition.cuh:61-116 (+ kernel partition_kernel.cuh:22-66).
 * d_segment_index: n x 3 (segment, slot, boundary slot or 0xffffffff); h_segment_start /
 * h_segment_length: centroid_num+1 entries, the last one is the boundary segment.
 * boundary_factor < 0 disables the boundary test (large path, partition_kernel.cuh:122-162).
 * Slots follow ascending row id (the reference's come from atomics and are arbitrary). */
int glide_define_partition(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, const float *d_centroids,
                           uint32_t centroid_num, float boundary_factor, int metric, uint32_t *d_segment_index,
                           uint32_t *h_segment_start, uint32_t *h_segment_length);
/* reorder, partition.cuh:118-157 (+ kernel partition_kernel.cuh:68-100).
 * d_reorder_data: (n + boundary) x dim, d_map: n + boundary. */
int glide_reorder(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, const uint32_t *d_segment_index,
                  const uint32_t *h_segment_start, uint32_t centroid_num, float *d_reorder_data, uint32_t *d_map);
/* preprocess, partition.cuh:159-193: the three steps above. The caller does not know the
 * boundary count in advance, so the outputs are allocated by the library (cudaMalloc) and
 * owned by the caller, who frees them with glide_free. */
int glide_preprocess(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, uint32_t centroid_num,
                     float boundary_factor, float sample_factor, int metric, uint64_t seed, float *d_centroids,
                     uint32_t *h_segment_start, uint32_t *h_segment_length, float **d_reorder_data_out,
                     uint32_t **d_map_out, uint32_t *reorder_num_out);
void glide_free(void *device_ptr);

/* ---- kNN stage -------------------------------------------------------------------------- */
/* build_nnd, nn_descent.cuh:1405-1467: per-partition kNN graph of the reordered rows,
 * partition-local ids, h_or_d knn: rows x knn_degree int32. knn_degree <= 64.
 * max_iterations 0 -> 20 and termination_threshold < 0 -> 1e-4 (params.cuh:20-21).
 * sample 0 -> 32. Partitions of at most exact_max_rows rows get their EXACT kNN graph from
 * an all-pairs kernel (cheaper than descent at that size); larger ones run NN-descent.
 * exact_max_rows 0xffffffff -> 16384, 0 -> NN-descent everywhere. */
int glide_build_nnd(glide_ctx *ctx, const float *d_reorder_data, uint32_t rows, uint32_t dim,
                    const uint32_t *h_segment_start, const uint32_t *h_segment_length, uint32_t segment_num,
                    uint32_t knn_degree, uint32_t max_iterations, float termination_threshold, uint32_t sample,
                    uint32_t exact_max_rows, uint64_t seed, int metric, int32_t *d_knn, uint32_t *iterations_run);
/* build_nnd for a run of whole partitions cut out of the reordered set (d_rows = the run's first row,
 * segment starts counted from that row): row_base is the run's first row within the whole set.
 * Seeds and padding depend on global row numbers, so the runs of a sharded build give exactly the
 * rows of one glide_build_nnd over everything. The reference runs one thread per partition on one
 * GPU (nn_descent.cuh:1304-1343); partitions are the unit a multi-GPU build hands to its ranks. */
int glide_build_nnd_range(glide_ctx *ctx, const float *d_rows, uint32_t rows, uint32_t dim,
                          const uint32_t *h_segment_start, const uint32_t *h_segment_length, uint32_t segment_num,
                          uint32_t knn_degree, uint32_t max_iterations, float termination_threshold, uint32_t sample,
                          uint32_t exact_max_rows, uint64_t seed, int metric, uint32_t row_base, int32_t *d_knn,
                          uint32_t *iterations_run);
/* Exact kNN by brute force: the ground truth (the reference reads it from a file,
 * small_search.cu:88). k <= 128. d_out_dists may be null. */
int glide_bruteforce_knn(glide_ctx *ctx, const float *d_base, uint32_t n, const float *d_queries, uint32_t q,
                         uint32_t dim, uint32_t k, int metric, uint32_t *d_out_ids, float *d_out_dists);

/* ---- graph build stage (glide_impl.cuh) ------------------------------------------------- */
/* start_point_select, glide_impl.cuh:43-73: one member per segment drawn from `seed`.
 * h_local: segment_num partition-local ids; h_original: centroid_num original ids. */
int glide_start_point_select(const uint32_t *h_segment_start, const uint32_t *h_segment_length,
                             uint32_t segment_num, const uint32_t *h_map, uint64_t seed, uint32_t *h_local,
                             uint32_t *h_original);
/* subgraph_build_and_merge, glide_impl.cuh:75-192: build_kernel over the `num` main rows
 * then build_boundary_kernel over the boundary copies. d_graph: num x graph_degree, every
 * slot must be 0xffffffff on entry. d_start_points_local: segment_num entries. */
int glide_subgraph_build_and_merge(glide_ctx *ctx, const float *d_reorder_data, uint32_t reorder_num, uint32_t dim,
                                   const uint32_t *d_knn, uint32_t knn_degree, const uint32_t *h_segment_start,
                                   const uint32_t *h_segment_length, uint32_t segment_num,
                                   const uint32_t *d_start_points_local, const uint32_t *d_map, uint32_t num,
                                   uint32_t graph_degree, const glide_search_params *p, float relaxant_factor,
                                   int metric, int skip_boundary, uint32_t *d_graph);
/* The same two kernels for reorder rows [first_row, first_row + row_count) only: rows below
 * `num` run build_kernel, rows from `num` on are boundary copies and run build_boundary_kernel
 * (the rows they merge into must already hold their build_kernel result). This is how the
 * build is sharded across GPUs; the reference launches whole ranges (glide_impl.cuh:114-187). */
int glide_subgraph_build_range(glide_ctx *ctx, const float *d_reorder_data, uint32_t reorder_num, uint32_t dim,
                               const uint32_t *d_knn, uint32_t knn_degree, const uint32_t *h_segment_start,
                               const uint32_t *h_segment_length, uint32_t segment_num,
                               const uint32_t *d_start_points_local, const uint32_t *d_map, uint32_t num,
                               uint32_t graph_degree, const glide_search_params *p, float relaxant_factor,
                               int metric, uint32_t first_row, uint32_t row_count, uint32_t *d_graph);
/* reverse_graph, glide_impl.cuh:194-256. In place. */
int glide_reverse_graph(glide_ctx *ctx, uint32_t *d_graph, uint32_t num, uint32_t graph_degree);
/* refine, glide_impl.cuh:258-317. In place. The reference's refine_kernel fills rows while other
 * CTAs still traverse them (graph_kernel.cuh:648, :660-671), so its result depends on the schedule;
 * here the points are taken in waves of 65,536 consecutive ids: a wave's searches read the rows the
 * earlier waves wrote, its own rows are written when the wave is done (same result on every run). */
int glide_refine(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph,
                 uint32_t graph_degree, const float *d_centroids, uint32_t centroid_num,
                 const uint32_t *d_start_points, const glide_search_params *p, float relaxant_factor, int metric);
/* glide_refine with the wave size given (0: one wave, every search reads the graph as it was before
 * the call). Same reference lines as glide_refine. */
int glide_refine_waves(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph,
                       uint32_t graph_degree, const float *d_centroids, uint32_t centroid_num,
                       const uint32_t *d_start_points, const glide_search_params *p, float relaxant_factor,
                       int metric, uint32_t wave_rows);

/* refine_kernel (glide_impl.cuh:284-312 launches the whole range) for points [first, first + count):
 * searches read d_graph, the refined rows go to d_rows_out (count x graph_degree, row of point p at
 * p - first); d_graph itself is not written. A rank of a sharded build refines its slice of a wave
 * this way and the slices are gathered before the wave is written back. */
int glide_refine_rows(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_graph,
                      uint32_t graph_degree, const float *d_centroids, uint32_t centroid_num,
                      const uint32_t *d_start_points, const glide_search_params *p, float relaxant_factor, int metric,
                      uint32_t first, uint32_t count, uint32_t *d_rows_out);
/* build_kernel (glide_impl.cuh:114-143) for the non-boundary reorder rows [first_row, first_row +
 * row_count): the row of reorder id r goes to d_rows_out at r - first_row (neighbours are original
 * ids, as in the finished graph) instead of to the row of its original id. Rows by reorder position
 * are contiguous per rank, which is what lets a sharded build exchange them with one all-gather. */
int glide_subgraph_build_rows(glide_ctx *ctx, const float *d_reorder_data, uint32_t reorder_num, uint32_t dim,
                              const uint32_t *d_knn, uint32_t knn_degree, const uint32_t *h_segment_start,
                              const uint32_t *h_segment_length, uint32_t segment_num,
                              const uint32_t *d_start_points_local, const uint32_t *d_map, uint32_t num,
                              uint32_t graph_degree, const glide_search_params *p, float relaxant_factor, int metric,
                              uint32_t first_row, uint32_t row_count, uint32_t *d_rows_out);

/* ---- communicator (multi-GPU builds and searches) -------------------------------------------
 * One process per GPU; the reference is a single-GPU program (its mains pin device 1,
 * small_build.cu:33) and has no counterpart for any of these. A context may carry one NCCL
 * communicator; collectives are enqueued on the context's stream, in order with its kernels.
 * libnccl.so.2 is opened at run time by the first of these calls. */
/* 128 opaque bytes made by one rank and carried to the others by the host (a file, a socket, MPI,
 * torch.distributed's store): the rendezvous token of glide_comm_init. */
int glide_comm_unique_id(uint8_t out[128]);
/* Collective: every rank calls it with the same id and world size. */
int glide_comm_init(glide_ctx *ctx, const uint8_t id[128], uint32_t world, uint32_t rank);
int glide_comm_destroy(glide_ctx *ctx);
uint32_t glide_comm_world(const glide_ctx *ctx);   /* 1 without a communicator */
uint32_t glide_comm_rank(const glide_ctx *ctx);
/* In-place all-gather of unequal blocks: rank r owns bytes [offsets[r], offsets[r] + counts[r]) of
 * d_buf (the same offsets and counts on every rank) and every rank ends with all blocks. Returns
 * after enqueueing. */
int glide_comm_all_gather_v(glide_ctx *ctx, void *d_buf, const uint64_t *offsets, const uint64_t *counts);
int glide_comm_broadcast(glide_ctx *ctx, void *d_buf, uint64_t bytes, uint32_t root);
/* Element-wise over the ranks, in place; op 0 sum, 1 max, 2 min. */
int glide_comm_all_reduce_u64(glide_ctx *ctx, uint64_t *d_buf, uint64_t count, int op);
/* Waits for everything enqueued on the context's stream (kernels, copies, collectives). */
int glide_ctx_synchronize(glide_ctx *ctx);

/* How many kNN stages of this context the tensor-core kernel gave back to the fp32 kernels (no
 * tensor map, a bounded wait that ran out, or more candidates at a row's threshold than its buffers
 * hold): 0 in normal operation; the results are correct either way. */
uint32_t glide_tc_knn_fallbacks(const glide_ctx *ctx);

/* ---- matrix files ----------------------------------------------------------------------- */
/* load_matrix_data, load.cuh:10-30 (u32 rows, u32 dim, then the rows; the reference reads row by
 * row into pageable memory). elem_bytes 4 (fp32, .fbin) or 1 (uint8). GLIDE_ERR_IO for a missing
 * file or one shorter than its header says. */
int glide_matrix_file_info(const char *path, uint32_t elem_bytes, uint32_t *rows, uint32_t *dim);
/* Reads rows [first_row, first_row + rows) of the file into h_rows (pin it: glide_host_alloc or
 * glide_host_register) with `threads` reader threads (0: 4) issuing positional reads of chunk_rows
 * rows (0: 64 MB worth). With d_centroids given, every chunk is uploaded and its rows assigned to
 * their nearest centroid (define_partition_for_large_kernel, partition_kernel.cuh:122-162) while
 * later chunks are still being read; h_nearest gets one partition id per row. Without centroids
 * the call only reads. stats (may be null): [0] seconds until the last chunk was in host memory,
 * [1] seconds until h_nearest was complete, [2] seconds the device side waited for the file. */
int glide_load_rows(glide_ctx *ctx, const char *path, uint32_t elem_bytes, uint64_t first_row, uint64_t rows, void *h_rows,
                    uint32_t chunk_rows, uint32_t threads, const float *d_centroids, uint32_t centroid_num, int metric,
                    uint32_t *h_nearest, double *stats);

/* ---- search stage ----------------------------------------------------------------------- */
/* GLIDE::search, glide_impl.cuh:370-454 (search_kernel, search_kernel.cuh:393-490).
 * Device pointers; results Q x top_k. */
int glide_search(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_graph,
                 uint32_t graph_degree, const float *d_centroids, uint32_t centroid_num,
                 const uint32_t *d_start_points, const float *d_queries, uint32_t q, const glide_search_params *p,
                 int metric, uint32_t *d_out_ids, float *d_out_dists);
/* Same call with HOST query and result buffers (copies inside), the shape of the
 * reference's small_search main (small_search.cu:113-117 upload, glide_impl.cuh:450-453
 * download). */
int glide_search_host(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_graph,
                      uint32_t graph_degree, const float *d_centroids, uint32_t centroid_num,
                      const uint32_t *d_start_points, const float *h_queries, uint32_t q,
                      const glide_search_params *p, int metric, uint32_t *h_out_ids, float *h_out_dists);
/* glide_search_host with several batches in flight (no counterpart in the reference, whose
 * small_search main blocks on every batch): uploads, kernels and downloads of consecutive batches
 * overlap. submit() enqueues one batch of at most max_queries queries from h_queries and returns
 * the slot it took; wait(slot) returns once that batch's results are in h_out_ids / h_out_dists.
 * Slots are taken in turn; submit() first waits for the batch that last used its slot. Host
 * buffers should be pinned (glide_host_alloc / glide_host_register), else the copies block.
 * Kernels run on the context's stream in submission order, so other calls on the context fall
 * in line behind them. */
typedef struct glide_search_pipe glide_search_pipe;
int glide_search_pipe_create(glide_ctx *ctx, uint32_t max_queries, uint32_t dim, uint32_t max_top_k, uint32_t depth,
                             glide_search_pipe **out);
void glide_search_pipe_destroy(glide_search_pipe *pipe);
int glide_search_pipe_submit(glide_search_pipe *pipe, const float *d_data, uint32_t num, uint32_t dim,
                             const uint32_t *d_graph, uint32_t graph_degree, const float *d_centroids,
                             uint32_t centroid_num, const uint32_t *d_start_points, const float *h_queries, uint32_t q,
                             const glide_search_params *p, int metric, uint32_t *h_out_ids, float *h_out_dists,
                             uint32_t *slot_out);
int glide_search_pipe_wait(glide_search_pipe *pipe, uint32_t slot);
/* glide_search for hosts that must not allocate at call time (a serving loop whose device
 * memory comes from its own pool and where a cudaMalloc would stall the device; a process
 * running near the memory limit). It has no counterpart in the reference. Same arguments and
 * results as glide_search; the per-query scratch (one word per query: the partition it is routed
 * to) is a fixed 256 KB array inside the library image, held by every GPU that loads the library
 * until the process exits, so at most 65,536 queries per call (more: GLIDE_ERR_UNSUPPORTED).
 * The call uses no cudaMalloc/cudaFree and no allocating library routine. The first call on a
 * device looks up the array's device address; make that call before starting any stream
 * capture. All calls on one device share the array (it needs no clearing: every word used is
 * written first), so two such calls that overlap on the GPU race; serialise them. */
int glide_search_static_scratch(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim,
                                const uint32_t *d_graph, uint32_t graph_degree, const float *d_centroids,
                                uint32_t centroid_num, const uint32_t *d_start_points, const float *d_queries,
                                uint32_t q, const glide_search_params *p, int metric, uint32_t *d_out_ids,
                                float *d_out_dists);
/* Device milliseconds of the two kernels of the last glide_search on this context:
 * out[0] the routing pre-pass (nearest centroid per query), out[1] the search kernel. */
void glide_last_search_split_ms(const glide_ctx *ctx, float out[2]);
/* Number of kernels the last glide_search enqueued (routing kernels + the search kernel). */
uint32_t glide_last_search_launches(const glide_ctx *ctx);
/* Counters of the last search/build/refine/define_partition call when enabled: rows read during
 * search, expansions, rows read during pruning, and a fourth that depends on the call: build and
 * refine count the points whose beam ended with fewer than `beam` entries; search and
 * define_partition count the points whose nearest centroid was settled by the exact
 * warp-per-point kernel (a tie, or too many candidates after the tensor-core prefilter). */
void glide_enable_counters(glide_ctx *ctx, int on);
int glide_read_counters(glide_ctx *ctx, uint64_t out[4]);

/* ---- large path (glide_large_impl.cuh) -------------------------------------------------- */
/* select_segment_kernel, search_kernel.cuh:546-607; d_out: q x centroid_num. */
int glide_select_segments(glide_ctx *ctx, const float *d_queries, uint32_t q, uint32_t dim,
                          const float *d_centroids, uint32_t centroid_num, uint32_t min_segment_num,
                          float boundary_factor, int metric, uint32_t *d_out);
/* search_on_sub_kernel, search_kernel.cuh:653-765: search one resident partition and fold
 * its results into the running top-k (d_final_*: q x top_k, initialised by the caller to
 * FLT_MAX / 0xffffffff before the first partition). */
int glide_search_on_sub(glide_ctx *ctx, const float *d_data, uint32_t dim, const uint32_t *d_graph,
                        uint32_t graph_degree, const uint32_t *d_map, uint32_t start_point,
                        const float *d_queries, uint32_t q, const uint32_t *d_segment_ids, uint32_t segment_num,
                        uint32_t segment_id, const glide_search_params *p, int metric, uint32_t *d_final_ids,
                        float *d_final_dists);
/* build_for_large_kernel / refine_for_large_kernel, graph_kernel.cuh:675-821: one resident
 * partition, local ids, no map. */
int glide_build_partition(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_knn,
                          uint32_t knn_degree, uint32_t start_point, uint32_t graph_degree,
                          const glide_search_params *p, float relaxant_factor, int metric, uint32_t *d_graph);
int glide_refine_partition(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph,
                           uint32_t graph_degree, uint32_t start_point, const glide_search_params *p,
                           float relaxant_factor, int metric);

/* ---- large path, host orchestration (GLIDE_large, glide_large.cuh:14-212) -----------------
 * The data set (reorder order) and the finished graph live in host memory that the caller has
 * pinned; partitions are streamed through two device slots with uploads, kernels and downloads on
 * three streams. Rows are fp32 (row_type 0) or uint8 (row_type 1, the reference's large-path type,
 * large_build.cu:84): bytes cross the host link and are widened to fp32 in HBM. */
typedef struct glide_large glide_large;
/* Page-locked host memory (cudaHostAlloc / cudaHostRegister), for hosts without a CUDA binding. */
int glide_host_alloc(size_t bytes, void **out);
void glide_host_free(void *p);
int glide_host_register(void *p, size_t bytes);
int glide_host_unregister(void *p);
/* GLIDE_large constructor, glide_large_impl.cuh:14-48: h_rows (segment s = rows
 * [h_segment_start[s], +h_segment_length[s])), h_map (reorder id -> original id) and h_graph
 * (rows x graph_degree, written by glide_large_build, read by glide_large_search) stay owned by
 * the caller and must outlive the object. One centroid per partition; segment_num <= 4096. */
int glide_large_create(glide_ctx *ctx, const void *h_rows, int row_type, uint32_t dim, const uint32_t *h_segment_start,
                       const uint32_t *h_segment_length, uint32_t segment_num, const uint32_t *h_map,
                       uint32_t graph_degree, int metric, uint32_t *h_graph, glide_large **out);
void glide_large_destroy(glide_large *index);
/* Partition-local start points (glide_large_impl.cuh:50-77): glide_large_build draws them (seeded);
 * an index loaded from stage files sets them. segment_num entries. */
int glide_large_set_start_points(glide_large *index, const uint32_t *h_start_points);
int glide_large_get_start_points(const glide_large *index, uint32_t *h_out);
/* GLIDE_large::build, glide_large_impl.cuh:79-328, for the listed partitions (a rank of a multi-GPU
 * build lists its own): kNN graph (NN-descent or the exact all-pairs kernel, as glide_build_nnd;
 * skipped when h_knn_in, rows x knn_degree partition-local ids, is given), build_for_large, reverse
 * edges, refine_for_large (p_refine null or beam 0: none). h_knn_out (pinned, may be null) receives
 * the kNN rows. Partition p + 1 is uploaded while p is built. Here and in the two calls below a null
 * partition_ids stands for every partition in index order (partition_count is then ignored). */
int glide_large_build(glide_large *index, const uint32_t *partition_ids, uint32_t partition_count, uint32_t knn_degree,
                      const glide_search_params *p_build, const glide_search_params *p_refine, float relaxant_factor,
                      uint32_t nnd_max_iterations, float nnd_termination_threshold, uint32_t nnd_sample,
                      uint32_t exact_max_rows, uint64_t seed, const int32_t *h_knn_in, int32_t *h_knn_out);
/* Keeps the listed partitions (fp32 rows, graph rows, id map) in device memory until budget_bytes
 * are used; searches then upload only the others. The reference uploads every partition for every
 * query batch (glide_large_impl.cuh:424-438). */
int glide_large_make_resident(glide_large *index, const uint32_t *partition_ids, uint32_t partition_count,
                              size_t budget_bytes, uint32_t *resident_count);
/* The device buffers of partition p as a resident partition (rows x dim fp32, rows x graph_degree ids,
 * rows ids), allocated uninitialised when p is not resident yet: for a rank that receives partitions
 * another rank built (glide_comm_broadcast into these buffers) and then searches them. */
int glide_large_resident_buffers(glide_large *index, uint32_t partition, float **d_rows, uint32_t **d_graph, uint32_t **d_map);
/* GLIDE_large::search, glide_large_impl.cuh:355-507, over the listed partitions (ascending index
 * order): routing (select_segment_kernel), then search_on_sub_kernel per partition that some query
 * of the batch is routed to. d_final_*: q x top_k, overwritten. */
int glide_large_search(glide_large *index, const float *d_queries, uint32_t q, const float *d_centroids,
                       uint32_t centroid_num, uint32_t min_segment_num, float boundary_factor,
                       const glide_search_params *p, const uint32_t *partition_ids, uint32_t partition_count,
                       uint32_t *d_final_ids, float *d_final_dists);
/* Merged index. GLIDE_large::build_with_merge is declared in the reference (glide_large.cuh:96) and
 * defined nowhere, so this is the library's own design, built from the large path's pieces: all
 * partitions in one piece of device memory (they must be resident), their subgraphs rewritten to
 * reorder ids, and links across partition borders: a point whose partitions within boundary_factor
 * of its nearest centroid (select_segment_kernel's rule) include others than its own is searched for
 * in those (p_link; p_link->top_k == link_count) and its link_count nearest finds enter its row
 * (holes first, then over the row's tail); reverse edges follow. stats (may be null): [0] seconds of
 * the link stage, [1] of the reverse edges, [2] rows that received links. */
int glide_large_merge(glide_large *index, const float *d_centroids, uint32_t centroid_num, float boundary_factor,
                      uint32_t link_count, const glide_search_params *p_link, double *stats);
/* One beam search per query over the merged graph (glide_search on it), entered at the nearest
 * centroid's start point; ids are original ids. */
int glide_large_search_merged(glide_large *index, const float *d_queries, uint32_t q, const float *d_centroids,
                              uint32_t centroid_num, const glide_search_params *p, uint32_t *d_out_ids, float *d_out_dists);
/* The merged graph, rows x graph_degree reorder ids, into host memory. */
int glide_large_merged_graph(const glide_large *index, uint32_t *h_out);
/* Statistics of the last glide_large_build / glide_large_search: out[0..3] kernel seconds (build: kNN,
 * subgraph build, reverse edges, refine; search: routing, per-partition search, 0, 0), out[4] bytes
 * uploaded, out[5] seconds from the first to the last upload on the upload stream, out[6] partitions
 * uploaded, out[7] partitions searched. */
void glide_large_last_stats(const glide_large *index, double out[8]);
/* result_merge (search_kernel.cuh:609-651) over whole result sets: folds `sets` result sets
 * (d_ids, d_dists: sets x q x top_k) into one, in set order. A multi-GPU search gathers the per-GPU
 * results and folds them with this. */
int glide_merge_results(glide_ctx *ctx, const uint32_t *d_ids, const float *d_dists, uint32_t sets, uint32_t q,
                        uint32_t top_k, uint32_t *d_out_ids, float *d_out_dists);

/* ---- device memory helpers for hosts without their own CUDA binding --------------------- */
int glide_malloc(glide_ctx *ctx, size_t bytes, void **d_out);
int glide_memcpy_h2d(glide_ctx *ctx, void *d_dst, const void *h_src, size_t bytes);
int glide_memcpy_d2h(glide_ctx *ctx, void *h_dst, const void *d_src, size_t bytes);
int glide_memset_u32(glide_ctx *ctx, uint32_t *d_dst, uint32_t value, size_t count);

#ifdef __cplusplus
}
#endif

#endif /* GLIDE_B200_H */
