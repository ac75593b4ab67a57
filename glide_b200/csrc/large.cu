// Large path: the data set and the finished graph live in (pinned) host memory, partitions pass
// through the GPU. Host orchestration of GLIDE_large (glide_large_impl.cuh:79-167 build, :169-328
// reverse and refine, :355-507 search), re-shaped for one B200:
//
//  * build: per partition H2D rows -> kNN graph -> build_for_large -> reverse edges -> refine ->
//    D2H rows of ids. Two device slots and three streams (upload, compute, download): partition
//    p + 1 is uploaded and partition p - 1 downloaded while p is being built. The reference
//    allocates, copies and frees per partition on one stream (:121-128, :164).
//  * rows may be uint8 in host memory (the reference's large path is uint8, large_build.cu:84):
//    they cross the host link as bytes and are widened to fp32 in HBM, where every kernel of the
//    small path serves them unchanged (integer-valued rows make this exact).
//  * search: residency is a policy. A B200 holds 180 GB, more than the whole 100M x 128 set, so
//    partitions (rows, graph rows, id map) are kept in HBM up to a byte budget and only the rest is
//    streamed per query batch; a partition is uploaded only if some query of the batch is routed to
//    it. The reference uploads every partition for every batch (:424-438).
//
// Every stage runs the same kernels as the per-partition entry points of the C ABI
// (glide_build_nnd_range, glide_build_partition, glide_reverse_graph, glide_refine_partition,
// glide_select_segments, glide_search_on_sub), so results equal theirs bit for bit.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/glide_b200.h"
#include "ctx.h"
#include "kernels.h"

namespace {

int fail(glide_ctx *ctx, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->error = buf;
    return code;
}

#define LG_CUDA(ctx, call)                                                                           \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ != cudaSuccess)                                                                       \
            return fail(ctx, e_ == cudaErrorMemoryAllocation ? GLIDE_ERR_NO_MEMORY : GLIDE_ERR_CUDA, \
                        "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__);        \
    } while (0)

__global__ void widen_u8_kernel(const uint8_t *__restrict__ in, float *__restrict__ out, size_t n4) {
    // four bytes in, one float4 out per thread
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const uchar4 b = reinterpret_cast<const uchar4 *>(in)[i];
    reinterpret_cast<float4 *>(out)[i] = make_float4((float) b.x, (float) b.y, (float) b.z, (float) b.w);
}

// a null partition list means every partition of the index, in index order
const uint32_t *every_partition(std::vector<uint32_t> &ids, uint32_t S, uint32_t *count) {
    ids.resize(S);
    for (uint32_t s = 0; s < S; s++) ids[s] = s;
    *count = S;
    return ids.data();
}

}  // namespace

namespace glide {
cudaError_t launch_widen_u8(const uint8_t *in, float *out, size_t count, cudaStream_t stream) {
    const size_t n4 = count / 4;
    if (n4 == 0) return cudaSuccess;
    widen_u8_kernel<<<(unsigned) ((n4 + 255) / 256), 256, 0, stream>>>(in, out, n4);
    return cudaGetLastError();
}
}  // namespace glide

namespace {

// routed[s] += number of queries whose list names partition s (lists end at the first 0xffffffff)
__global__ void count_routed_kernel(const uint32_t *__restrict__ segment_ids, uint32_t Q, uint32_t C, uint32_t *routed) {
    const uint32_t q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= Q) return;
    for (uint32_t i = 0; i < C; i++) {
        const uint32_t s = segment_ids[(size_t) q * C + i];
        if (s == 0xffffffffu) break;
        if (s < C) atomicAdd(routed + s, 1u);
    }
}

// result_merge (search_kernel.cuh:609-651) applied to whole result sets: out starts as set 0 and sets
// 1 .. G-1 are folded into it in order, each with the reference's network of width M (a power of two
// >= top_k, >= 32): position j of the running list is compared with position M-1-j of the incoming
// one, the incoming entry wins only when strictly nearer, then one bitonic merge phase that never
// exchanges equal keys. A warp per query; mk/mv: M words each per warp.
__global__ void __launch_bounds__(128) merge_results_kernel(const uint32_t *__restrict__ ids, const float *__restrict__ dists,
                                                            uint32_t G, uint32_t Q, uint32_t top_k, uint32_t M,
                                                            uint32_t *out_ids, float *out_dists) {
    extern __shared__ __align__(16) uint32_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t q = blockIdx.x * (blockDim.x >> 5) + warp;
    if (q >= Q) return;
    float *mk = reinterpret_cast<float *>(smem) + (size_t) warp * 2 * M;
    uint32_t *mv = reinterpret_cast<uint32_t *>(mk + M);
    const size_t set = (size_t) Q * top_k;
    for (uint32_t j = lane; j < M; j += 32) {
        mk[j] = j < top_k ? dists[(size_t) q * top_k + j] : 3.402823466e+38f;
        mv[j] = j < top_k ? ids[(size_t) q * top_k + j] : 0xffffffffu;
    }
    __syncwarp();
    for (uint32_t g = 1; g < G; g++) {
        const float *rk = dists + g * set + (size_t) q * top_k;
        const uint32_t *rv = ids + g * set + (size_t) q * top_k;
        for (uint32_t j = lane; j < M; j += 32) {
            const uint32_t k = M - 1 - j;
            if (k < top_k && mk[j] > rk[k]) { mk[j] = rk[k]; mv[j] = rv[k]; }
        }
        __syncwarp();
        for (uint32_t stride = M >> 1; stride >= 1; stride >>= 1) {
            for (uint32_t p = lane; p < M / 2; p += 32) {
                const uint32_t lo = ((p / stride) * 2 * stride) + (p % stride), hi = lo + stride;
                const float k0 = mk[lo], k1 = mk[hi];
                if ((k0 != k1) && !(k0 < k1)) {
                    mk[lo] = k1; mk[hi] = k0;
                    const uint32_t t = mv[lo]; mv[lo] = mv[hi]; mv[hi] = t;
                }
            }
            __syncwarp();
        }
        // entries past top_k do not survive a merge (the reference writes back top_k entries and
        // re-pads the list for the next partition)
        for (uint32_t j = top_k + lane; j < M; j += 32) { mk[j] = 3.402823466e+38f; mv[j] = 0xffffffffu; }
        __syncwarp();
    }
    for (uint32_t j = lane; j < top_k; j += 32) {
        out_dists[(size_t) q * top_k + j] = mk[j];
        out_ids[(size_t) q * top_k + j] = mv[j];
    }
}

// ---- merged index ------------------------------------------------------------------------------
__global__ void iota_kernel(uint32_t *out, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = i;
}

// partition-local ids -> reorder ids
__global__ void globalise_kernel(const uint32_t *__restrict__ local, size_t entries, uint32_t offset, uint32_t *__restrict__ out) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= entries) return;
    const uint32_t v = local[i];
    out[i] = v == 0xffffffffu ? v : v + offset;
}

// A data point's list of partitions within the boundary factor, without the partition it lives in
// (row r of the chunk is reorder id first_row + r; lists end at the first 0xffffffff).
__global__ void drop_own_kernel(uint32_t *routes, uint32_t rows, uint32_t S, uint32_t first_row, const uint32_t *__restrict__ seg_start) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const uint32_t id = first_row + r;
    uint32_t lo = 0, hi = S;                       // last partition whose start is <= id
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (seg_start[mid] <= id) lo = mid; else hi = mid;
    }
    uint32_t *list = routes + (size_t) r * S;
    uint32_t kept = 0;
    for (uint32_t i = 0; i < S; i++) {
        const uint32_t s = list[i];
        if (s == 0xffffffffu) break;
        if (s != lo) list[kept++] = s;
    }
    for (uint32_t i = kept; i < S && list[i] != 0xffffffffu; i++) list[i] = 0xffffffffu;
}

// Links into a row: every link id (nearest first, the list ends at 0xffffffff) that the row does not
// hold yet goes into the row's first hole, or, when there is none, over the last entry that is not
// itself a link of this pass (rows are in pick order, so the tail holds the least wanted edges).
__global__ void link_merge_kernel(uint32_t *graph_rows, const uint32_t *__restrict__ links, uint32_t rows, uint32_t degree,
                                  uint32_t link_count, uint32_t *rows_with_links) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    uint32_t *row = graph_rows + (size_t) r * degree;
    const uint32_t *mine = links + (size_t) r * link_count;
    uint32_t placed[8] = {0, 0, 0, 0, 0, 0, 0, 0};   // positions written in this pass (degree <= 256)
    uint32_t tail = degree, any = 0;
    for (uint32_t l = 0; l < link_count; l++) {
        const uint32_t id = mine[l];
        if (id == 0xffffffffu) break;
        bool have = false;
        uint32_t hole = degree;
        for (uint32_t i = 0; i < degree; i++) {
            const uint32_t e = row[i];
            if (e == id) { have = true; break; }
            if (e == 0xffffffffu && hole == degree) hole = i;
        }
        if (have) continue;
        uint32_t pos = hole;
        if (pos == degree) {
            while (tail > 0 && ((placed[(tail - 1) >> 5] >> ((tail - 1) & 31u)) & 1u)) tail--;
            if (tail == 0) break;
            pos = --tail;
        }
        row[pos] = id;
        placed[pos >> 5] |= 1u << (pos & 31u);
        any = 1;
    }
    if (any) atomicAdd(rows_with_links, 1u);
}

__global__ void map_ids_kernel(uint32_t *ids, const uint32_t *__restrict__ map, size_t count) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t v = ids[i];
    if (v != 0xffffffffu) ids[i] = map[v];
}

struct Slot {   // one partition's worth of device memory
    void *raw = nullptr;        // uint8 rows as uploaded (only for uint8 sets)
    float *rows = nullptr;      // fp32 rows the kernels read
    uint32_t *graph = nullptr;
    uint32_t *map = nullptr;
    int32_t *knn = nullptr;
    cudaEvent_t uploaded = nullptr, computed = nullptr, downloaded = nullptr;
    bool view = false;          // rows and map point into the merged index's arena and are not this slot's to free
};

}  // namespace

struct glide_large {
    glide_ctx *ctx = nullptr;
    const void *h_rows = nullptr;   // pinned host memory, reorder order
    int row_type = 0;               // 0 fp32, 1 uint8
    uint32_t dim = 0, degree = 0;
    int metric = 0;
    std::vector<uint32_t> seg_start, seg_len, start_points;
    const uint32_t *h_map = nullptr;
    uint32_t *h_graph = nullptr;    // pinned host memory, rows at reorder position
    cudaStream_t up = nullptr, down = nullptr;
    Slot slot[2];
    uint32_t slot_rows = 0;         // capacity of a slot, rows
    bool slot_has_knn = false;
    std::vector<Slot> resident;     // per partition; rows == nullptr when not resident
    size_t resident_bytes = 0;
    glide::PartitionRef *d_parts = nullptr;   // S entries: where each resident partition lies in device memory
    uint32_t *d_routed = nullptr;   // S counters
    uint32_t *d_routes = nullptr;   // Q x S
    size_t routes_capacity = 0;
    // merged index (glide_large_merge): every partition in one piece of device memory, one graph over
    // reorder ids with links across partition borders
    float *arena_rows = nullptr;        // n x dim
    uint32_t *merged_graph = nullptr;   // n x degree, reorder ids
    uint32_t *arena_map = nullptr;      // n: reorder id -> original id
    uint32_t *d_gid = nullptr;          // n: 0, 1, 2, ... (the id map of the link search: results in reorder ids)
    uint32_t *d_start_global = nullptr; // S: every partition's start point as a reorder id
    uint32_t *d_seg_start = nullptr;    // S
    double last_h2d_bytes = 0, last_h2d_seconds = 0;
    float last_stage_seconds[4] = {0, 0, 0, 0};   // kNN, build, reverse, refine (kernel time)
    uint32_t last_uploaded_partitions = 0, last_searched_partitions = 0;

    size_t row_bytes() const { return (size_t) dim * (row_type == 1 ? 1 : 4); }
};

namespace {

void free_slot(Slot &s) {
    if (s.raw) cudaFree(s.raw);
    if (s.rows && !s.view) cudaFree(s.rows);
    if (s.graph) cudaFree(s.graph);
    if (s.map && !s.view) cudaFree(s.map);
    if (s.knn) cudaFree(s.knn);
    if (s.uploaded) cudaEventDestroy(s.uploaded);
    if (s.computed) cudaEventDestroy(s.computed);
    if (s.downloaded) cudaEventDestroy(s.downloaded);
    s = Slot();
}

int alloc_slot(glide_large *L, Slot &s, uint32_t rows, bool with_knn, uint32_t knn_degree, bool with_events) {
    glide_ctx *ctx = L->ctx;
    if (L->row_type == 1) LG_CUDA(ctx, cudaMalloc(&s.raw, (size_t) rows * L->dim));
    LG_CUDA(ctx, cudaMalloc(&s.rows, (size_t) rows * L->dim * 4));
    LG_CUDA(ctx, cudaMalloc(&s.graph, (size_t) rows * L->degree * 4));
    LG_CUDA(ctx, cudaMalloc(&s.map, (size_t) rows * 4));
    if (with_knn) LG_CUDA(ctx, cudaMalloc(&s.knn, (size_t) rows * knn_degree * 4));
    if (with_events) {
        LG_CUDA(ctx, cudaEventCreateWithFlags(&s.uploaded, cudaEventDisableTiming));
        LG_CUDA(ctx, cudaEventCreateWithFlags(&s.computed, cudaEventDisableTiming));
        LG_CUDA(ctx, cudaEventCreateWithFlags(&s.downloaded, cudaEventDisableTiming));
    }
    return GLIDE_OK;
}

int ensure_slots(glide_large *L, uint32_t rows, bool with_knn, uint32_t knn_degree) {
    if (L->slot[0].rows && L->slot_rows >= rows && (!with_knn || L->slot_has_knn)) return GLIDE_OK;
    cudaStreamSynchronize(L->up);
    cudaStreamSynchronize(L->down);
    cudaStreamSynchronize(L->ctx->stream);
    for (auto &s : L->slot) free_slot(s);
    for (auto &s : L->slot) {
        int rc = alloc_slot(L, s, rows, with_knn, knn_degree, true);
        if (rc) return rc;
    }
    L->slot_rows = rows;
    L->slot_has_knn = with_knn;
    return GLIDE_OK;
}

// rows of partition p -> slot, on stream `st`; the widening kernel runs on the same stream
int upload_rows(glide_large *L, uint32_t p, Slot &s, cudaStream_t st) {
    glide_ctx *ctx = L->ctx;
    const size_t len = L->seg_len[p];
    const char *src = static_cast<const char *>(L->h_rows) + (size_t) L->seg_start[p] * L->row_bytes();
    if (L->row_type == 1) {
        LG_CUDA(ctx, cudaMemcpyAsync(s.raw, src, len * L->dim, cudaMemcpyHostToDevice, st));
        const size_t n4 = len * L->dim / 4;
        widen_u8_kernel<<<(unsigned) ((n4 + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t *>(s.raw), s.rows, n4);
        LG_CUDA(ctx, cudaGetLastError());
    } else {
        LG_CUDA(ctx, cudaMemcpyAsync(s.rows, src, len * L->dim * 4, cudaMemcpyHostToDevice, st));
    }
    return GLIDE_OK;
}

}  // namespace

extern "C" {

int glide_host_alloc(size_t bytes, void **out) {
    if (!out) return GLIDE_ERR_BAD_ARG;
    return cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocPortable) == cudaSuccess ? GLIDE_OK : GLIDE_ERR_NO_MEMORY;
}
void glide_host_free(void *p) { if (p) cudaFreeHost(p); }
int glide_host_register(void *p, size_t bytes) {
    if (!p) return GLIDE_ERR_BAD_ARG;
    return cudaHostRegister(p, bytes, cudaHostRegisterPortable) == cudaSuccess ? GLIDE_OK : GLIDE_ERR_CUDA;
}
int glide_host_unregister(void *p) { return (p && cudaHostUnregister(p) == cudaSuccess) ? GLIDE_OK : GLIDE_ERR_CUDA; }

// Folds G result sets (d_ids, d_dists: G x q x top_k, set g at offset g*q*top_k; each set sorted
// ascending and padded with (FLT_MAX, 0xffffffff)) into one, in set order: what a multi-GPU search
// does with the per-GPU results after gathering them.
int glide_merge_results(glide_ctx *ctx, const uint32_t *d_ids, const float *d_dists, uint32_t sets, uint32_t q,
                        uint32_t top_k, uint32_t *d_out_ids, float *d_out_dists) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (!d_ids || !d_dists || !d_out_ids || !d_out_dists || sets == 0) return fail(ctx, GLIDE_ERR_BAD_ARG, "merge_results: bad argument");
    if (top_k == 0 || top_k > 128) return fail(ctx, GLIDE_ERR_UNSUPPORTED, "Unsupported topk");   // kernel_config.cuh:309-319
    if (q == 0) return GLIDE_OK;
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    const uint32_t M = top_k <= 32 ? 32 : (top_k <= 64 ? 64 : 128);
    const uint32_t warps = 4;
    merge_results_kernel<<<(q + warps - 1) / warps, warps * 32, (size_t) warps * 2 * M * 4, ctx->stream>>>(
        d_ids, d_dists, sets, q, top_k, M, d_out_ids, d_out_dists);
    LG_CUDA(ctx, cudaGetLastError());
    LG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return GLIDE_OK;
}

int glide_large_create(glide_ctx *ctx, const void *h_rows, int row_type, uint32_t dim, const uint32_t *h_segment_start,
                       const uint32_t *h_segment_length, uint32_t segment_num, const uint32_t *h_map,
                       uint32_t graph_degree, int metric, uint32_t *h_graph, glide_large **out) {
    if (!ctx || !out) return GLIDE_ERR_BAD_ARG;
    *out = nullptr;
    if (!h_rows || !h_segment_start || !h_segment_length || !h_map || !h_graph || segment_num == 0 || dim == 0)
        return fail(ctx, GLIDE_ERR_BAD_ARG, "large_create: null pointer or zero size");
    if (row_type != 0 && row_type != 1) return fail(ctx, GLIDE_ERR_UNSUPPORTED, "large_create: rows must be fp32 (0) or uint8 (1)");
    if (row_type == 1 && dim % 4) return fail(ctx, GLIDE_ERR_UNSUPPORTED, "large_create: uint8 rows need dim % 4 == 0");
    if (graph_degree == 0 || graph_degree > 256) return fail(ctx, GLIDE_ERR_UNSUPPORTED, "Unsupported graph_degree");
    if (segment_num > 4096) return fail(ctx, GLIDE_ERR_UNSUPPORTED, "Unsupported centroid_size");
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    glide_large *L = new (std::nothrow) glide_large();
    if (!L) return GLIDE_ERR_NO_MEMORY;
    L->ctx = ctx; L->h_rows = h_rows; L->row_type = row_type; L->dim = dim; L->degree = graph_degree; L->metric = metric;
    L->seg_start.assign(h_segment_start, h_segment_start + segment_num);
    L->seg_len.assign(h_segment_length, h_segment_length + segment_num);
    L->start_points.assign(segment_num, 0);
    L->h_map = h_map; L->h_graph = h_graph;
    L->resident.resize(segment_num);
    if (cudaStreamCreateWithFlags(&L->up, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&L->down, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&L->d_routed, (size_t) segment_num * 4) != cudaSuccess ||
        cudaMalloc(&L->d_parts, (size_t) segment_num * sizeof(glide::PartitionRef)) != cudaSuccess) {
        glide_large_destroy(L);
        return fail(ctx, GLIDE_ERR_CUDA, "large_create: stream or counter allocation failed");
    }
    *out = L;
    return GLIDE_OK;
}

void glide_large_destroy(glide_large *L) {
    if (!L) return;
    cudaSetDevice(L->ctx->device);
    if (L->up) cudaStreamSynchronize(L->up);
    if (L->down) cudaStreamSynchronize(L->down);
    cudaStreamSynchronize(L->ctx->stream);
    for (auto &s : L->slot) free_slot(s);
    for (auto &s : L->resident) free_slot(s);
    if (L->d_routed) cudaFree(L->d_routed);
    if (L->d_parts) cudaFree(L->d_parts);
    if (L->d_routes) cudaFree(L->d_routes);
    cudaFree(L->arena_rows); cudaFree(L->merged_graph); cudaFree(L->arena_map); cudaFree(L->d_gid);
    cudaFree(L->d_start_global); cudaFree(L->d_seg_start);
    if (L->up) cudaStreamDestroy(L->up);
    if (L->down) cudaStreamDestroy(L->down);
    delete L;
}

int glide_large_set_start_points(glide_large *L, const uint32_t *h_start_points) {
    if (!L || !h_start_points) return GLIDE_ERR_BAD_ARG;
    std::copy(h_start_points, h_start_points + L->start_points.size(), L->start_points.begin());
    return GLIDE_OK;
}
int glide_large_get_start_points(const glide_large *L, uint32_t *h_out) {
    if (!L || !h_out) return GLIDE_ERR_BAD_ARG;
    std::copy(L->start_points.begin(), L->start_points.end(), h_out);
    return GLIDE_OK;
}

// Statistics of the last build or search call: out[0..3] kernel seconds of kNN, subgraph build, reverse
// edges, refine (build) or of routing and per-partition search in out[0], out[1] (search); out[4] bytes
// uploaded, out[5] seconds the uploads took end to end on their stream, out[6] partitions uploaded,
// out[7] partitions searched.
void glide_large_last_stats(const glide_large *L, double out[8]) {
    if (!L || !out) return;
    for (int i = 0; i < 4; i++) out[i] = L->last_stage_seconds[i];
    out[4] = L->last_h2d_bytes; out[5] = L->last_h2d_seconds;
    out[6] = L->last_uploaded_partitions; out[7] = L->last_searched_partitions;
}

int glide_large_build(glide_large *L, const uint32_t *partition_ids, uint32_t partition_count, uint32_t knn_degree,
                      const glide_search_params *p_build, const glide_search_params *p_refine, float relaxant_factor,
                      uint32_t nnd_max_iterations, float nnd_termination_threshold, uint32_t nnd_sample,
                      uint32_t exact_max_rows, uint64_t seed, const int32_t *h_knn_in, int32_t *h_knn_out) {
    if (!L) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = L->ctx;
    if (!p_build) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_build: null pointer");
    if (knn_degree == 0 || knn_degree > 64) return fail(ctx, GLIDE_ERR_UNSUPPORTED, "large_build: knn_degree must be <= 64");
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    const uint32_t S = (uint32_t) L->seg_len.size();
    std::vector<uint32_t> every;
    if (!partition_ids) partition_ids = every_partition(every, S, &partition_count);
    uint32_t max_rows = 0;
    for (uint32_t i = 0; i < partition_count; i++) {
        if (partition_ids[i] >= S) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_build: partition id out of range");
        max_rows = std::max(max_rows, L->seg_len[partition_ids[i]]);
    }
    for (auto &t : L->last_stage_seconds) t = 0;
    L->last_h2d_bytes = 0; L->last_h2d_seconds = 0; L->last_uploaded_partitions = 0; L->last_searched_partitions = 0;
    if (max_rows == 0) return GLIDE_OK;
    int rc = ensure_slots(L, max_rows, true, knn_degree);
    if (rc) return rc;
    // seeded start points, one per partition (glide_large_impl.cuh:50-77 draws them unseeded)
    {
        uint64_t x = seed;
        std::vector<uint64_t> draws(S);
        for (uint32_t s = 0; s < S; s++) {   // one draw per partition in partition order, whichever subset is built here
            uint64_t z = (x += 0x9E3779B97F4A7C15ull);
            z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
            z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
            draws[s] = z ^ (z >> 31);
        }
        for (uint32_t i = 0; i < partition_count; i++) {
            const uint32_t p = partition_ids[i];
            L->start_points[p] = L->seg_len[p] ? (uint32_t) (draws[p] % L->seg_len[p]) : 0;
        }
    }
    cudaEvent_t up_begin, up_end;
    LG_CUDA(ctx, cudaEventCreate(&up_begin));
    LG_CUDA(ctx, cudaEventCreate(&up_end));
    float up_ms_total = 0;
    auto upload = [&](uint32_t i) -> int {
        const uint32_t p = partition_ids[i];
        Slot &s = L->slot[i & 1];
        if (L->seg_len[p] == 0) { cudaEventRecord(s.uploaded, L->up); return GLIDE_OK; }
        // the slot is free once the partition that used it two steps ago has been downloaded
        LG_CUDA(ctx, cudaStreamWaitEvent(L->up, s.downloaded, 0));
        int r = upload_rows(L, p, s, L->up);
        if (r) return r;
        if (h_knn_in)
            LG_CUDA(ctx, cudaMemcpyAsync(s.knn, h_knn_in + (size_t) L->seg_start[p] * knn_degree,
                                         (size_t) L->seg_len[p] * knn_degree * 4, cudaMemcpyHostToDevice, L->up));
        LG_CUDA(ctx, cudaEventRecord(s.uploaded, L->up));
        L->last_h2d_bytes += (double) L->seg_len[p] * (L->row_bytes() + (h_knn_in ? knn_degree * 4.0 : 0.0));
        L->last_uploaded_partitions++;
        return GLIDE_OK;
    };
    for (auto &s : L->slot) LG_CUDA(ctx, cudaEventRecord(s.downloaded, L->down));
    LG_CUDA(ctx, cudaEventRecord(up_begin, L->up));
    rc = upload(0);
    for (uint32_t i = 0; i < partition_count && rc == GLIDE_OK; i++) {
        const uint32_t p = partition_ids[i];
        const uint32_t len = L->seg_len[p];
        Slot &s = L->slot[i & 1];
        if (i + 1 < partition_count) rc = upload(i + 1);   // rides under this partition's kernels
        if (rc || len == 0) continue;
        LG_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, s.uploaded, 0));
        if (!h_knn_in) {
            const uint32_t zero = 0;
            rc = glide_build_nnd_range(ctx, s.rows, len, L->dim, &zero, &len, 1, knn_degree, nnd_max_iterations,
                                       nnd_termination_threshold, nnd_sample, exact_max_rows, seed, L->metric,
                                       L->seg_start[p], s.knn, nullptr);
            if (rc) break;
            L->last_stage_seconds[0] += ctx->last_ms / 1e3f;
        }
        rc = glide_build_partition(ctx, s.rows, len, L->dim, reinterpret_cast<const uint32_t *>(s.knn), knn_degree,
                                   L->start_points[p], L->degree, p_build, relaxant_factor, L->metric, s.graph);
        if (rc) break;
        L->last_stage_seconds[1] += ctx->last_ms / 1e3f;
        rc = glide_reverse_graph(ctx, s.graph, len, L->degree);
        if (rc) break;
        L->last_stage_seconds[2] += ctx->last_ms / 1e3f;
        if (p_refine && p_refine->beam != 0) {
            rc = glide_refine_partition(ctx, s.rows, len, L->dim, s.graph, L->degree, L->start_points[p], p_refine,
                                        relaxant_factor, L->metric);
            if (rc) break;
            L->last_stage_seconds[3] += ctx->last_ms / 1e3f;
        }
        LG_CUDA(ctx, cudaEventRecord(s.computed, ctx->stream));
        LG_CUDA(ctx, cudaStreamWaitEvent(L->down, s.computed, 0));
        LG_CUDA(ctx, cudaMemcpyAsync(L->h_graph + (size_t) L->seg_start[p] * L->degree, s.graph, (size_t) len * L->degree * 4,
                                     cudaMemcpyDeviceToHost, L->down));
        if (h_knn_out)
            LG_CUDA(ctx, cudaMemcpyAsync(h_knn_out + (size_t) L->seg_start[p] * knn_degree, s.knn,
                                         (size_t) len * knn_degree * 4, cudaMemcpyDeviceToHost, L->down));
        LG_CUDA(ctx, cudaEventRecord(s.downloaded, L->down));
    }
    cudaEventRecord(up_end, L->up);
    cudaStreamSynchronize(L->up);
    cudaStreamSynchronize(L->down);
    cudaStreamSynchronize(ctx->stream);
    cudaEventElapsedTime(&up_ms_total, up_begin, up_end);
    L->last_h2d_seconds = up_ms_total / 1e3;
    cudaEventDestroy(up_begin);
    cudaEventDestroy(up_end);
    return rc;
}

// Keeps partitions (rows widened to fp32, graph rows, id map) in HBM, in the order given, until
// budget_bytes are used; partitions already resident stay. Returns how many of the listed ones are
// resident afterwards in *resident_count.
int glide_large_make_resident(glide_large *L, const uint32_t *partition_ids, uint32_t partition_count, size_t budget_bytes,
                              uint32_t *resident_count) {
    if (!L) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = L->ctx;
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    std::vector<uint32_t> every;
    if (!partition_ids) partition_ids = every_partition(every, (uint32_t) L->seg_len.size(), &partition_count);
    uint32_t n = 0;
    for (uint32_t i = 0; i < partition_count; i++) {
        const uint32_t p = partition_ids[i];
        if (p >= L->seg_len.size()) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_make_resident: partition id out of range");
        Slot &s = L->resident[p];
        const uint32_t len = L->seg_len[p];
        if (s.rows) { n++; continue; }
        if (len == 0) continue;
        const size_t need = (size_t) len * (L->dim * 4 + L->degree * 4 + 4) + (L->row_type == 1 ? (size_t) len * L->dim : 0);
        if (L->resident_bytes + need > budget_bytes) continue;
        int rc = alloc_slot(L, s, len, false, 0, false);
        if (rc) { free_slot(s); return rc; }
        rc = upload_rows(L, p, s, L->up);
        if (rc) return rc;
        LG_CUDA(ctx, cudaMemcpyAsync(s.graph, L->h_graph + (size_t) L->seg_start[p] * L->degree, (size_t) len * L->degree * 4,
                                     cudaMemcpyHostToDevice, L->up));
        LG_CUDA(ctx, cudaMemcpyAsync(s.map, L->h_map + L->seg_start[p], (size_t) len * 4, cudaMemcpyHostToDevice, L->up));
        if (s.raw) {   // the byte copy is only a staging area
            LG_CUDA(ctx, cudaStreamSynchronize(L->up));
            cudaFree(s.raw);
            s.raw = nullptr;
        }
        L->resident_bytes += (size_t) len * (L->dim * 4 + L->degree * 4 + 4);
        n++;
    }
    LG_CUDA(ctx, cudaStreamSynchronize(L->up));
    if (resident_count) *resident_count = n;
    return GLIDE_OK;
}

// Device buffers of partition p as a resident partition, allocated here when it is not resident yet
// and then left for the caller to fill: a rank that searches partitions another rank built receives
// their rows (fp32), graph rows and id map over NCCL straight into these buffers.
int glide_large_resident_buffers(glide_large *L, uint32_t p, float **d_rows, uint32_t **d_graph, uint32_t **d_map) {
    if (!L || !d_rows || !d_graph || !d_map) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = L->ctx;
    if (p >= L->seg_len.size()) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_resident_buffers: partition id out of range");
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    Slot &s = L->resident[p];
    const uint32_t len = L->seg_len[p];
    if (!s.rows && len) {
        int rc = alloc_slot(L, s, len, false, 0, false);
        if (rc) { free_slot(s); return rc; }
        if (s.raw) { cudaFree(s.raw); s.raw = nullptr; }   // the caller delivers fp32 rows
        L->resident_bytes += (size_t) len * (L->dim * 4 + L->degree * 4 + 4);
    }
    *d_rows = s.rows; *d_graph = s.graph; *d_map = s.map;
    return GLIDE_OK;
}

int glide_large_search(glide_large *L, const float *d_queries, uint32_t q, const float *d_centroids, uint32_t centroid_num,
                       uint32_t min_segment_num, float boundary_factor, const glide_search_params *p,
                       const uint32_t *partition_ids, uint32_t partition_count, uint32_t *d_final_ids,
                       float *d_final_dists) {
    if (!L) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = L->ctx;
    if (!d_queries || !d_centroids || !p || !d_final_ids || !d_final_dists)
        return fail(ctx, GLIDE_ERR_BAD_ARG, "large_search: null pointer");
    const uint32_t S = (uint32_t) L->seg_len.size();
    std::vector<uint32_t> every;
    if (!partition_ids) partition_ids = every_partition(every, S, &partition_count);
    if (centroid_num != S) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_search: one centroid per partition expected");
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    for (auto &t : L->last_stage_seconds) t = 0;
    L->last_h2d_bytes = 0; L->last_h2d_seconds = 0; L->last_uploaded_partitions = 0; L->last_searched_partitions = 0;
    if (q == 0) return GLIDE_OK;
    if ((size_t) q * S > L->routes_capacity) {
        if (L->d_routes) cudaFree(L->d_routes);
        L->d_routes = nullptr;
        LG_CUDA(ctx, cudaMalloc(&L->d_routes, (size_t) q * S * 4));
        L->routes_capacity = (size_t) q * S;
    }
    // the running result starts empty (glide_large_impl.cuh:376-379)
    LG_CUDA(ctx, cudaMemsetAsync(d_final_ids, 0xff, (size_t) q * p->top_k * 4, ctx->stream));
    {
        std::vector<float> init((size_t) q * p->top_k, 3.402823466e+38f);
        LG_CUDA(ctx, cudaMemcpyAsync(d_final_dists, init.data(), init.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        LG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    int rc = glide_select_segments(ctx, d_queries, q, L->dim, d_centroids, S, min_segment_num, boundary_factor, L->metric, L->d_routes);
    if (rc) return rc;
    L->last_stage_seconds[0] = ctx->last_ms / 1e3f;
    LG_CUDA(ctx, cudaMemsetAsync(L->d_routed, 0, (size_t) S * 4, ctx->stream));
    count_routed_kernel<<<(q + 255) / 256, 256, 0, ctx->stream>>>(L->d_routes, q, S, L->d_routed);
    LG_CUDA(ctx, cudaGetLastError());
    std::vector<uint32_t> routed(S);
    LG_CUDA(ctx, cudaMemcpyAsync(routed.data(), L->d_routed, (size_t) S * 4, cudaMemcpyDeviceToHost, ctx->stream));
    LG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // partitions of this call that some query visits, in index order (the order fixes how ties merge)
    std::vector<uint32_t> todo;
    uint32_t max_stream_rows = 0;
    for (uint32_t i = 0; i < partition_count; i++) {
        const uint32_t s = partition_ids[i];
        if (s >= S) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_search: partition id out of range");
        if (routed[s] == 0 || L->seg_len[s] == 0) continue;
        todo.push_back(s);
        if (!L->resident[s].rows) max_stream_rows = std::max(max_stream_rows, L->seg_len[s]);
    }
    std::sort(todo.begin(), todo.end());
    if (max_stream_rows == 0 && !todo.empty()) {
        // Every partition this batch visits lies in device memory: one launch, a warp per query walks
        // the partitions the query is routed to in ascending order (the order of the reference's
        // loop over partitions), instead of one launch per partition in which most warps find that
        // their query is not routed there.
        std::vector<glide::PartitionRef> refs(S, glide::PartitionRef{nullptr, nullptr, nullptr, 0, 0});
        for (uint32_t s : todo) {
            const Slot &r = L->resident[s];
            refs[s] = glide::PartitionRef{r.rows, r.graph, r.map, L->start_points[s], L->seg_len[s]};
        }
        LG_CUDA(ctx, cudaMemcpyAsync(L->d_parts, refs.data(), (size_t) S * sizeof(glide::PartitionRef), cudaMemcpyHostToDevice, ctx->stream));
        LG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // refs is a local vector
        if (p->beam < 32 || p->beam % 32 || p->beam > 512 || p->top_k < 1 || p->top_k > 128 || p->top_k > p->beam)
            return fail(ctx, GLIDE_ERR_BAD_ARG, "large_search: bad search parameters");
        glide::SearchArgs a{};
        a.degree = L->degree; a.dim = L->dim; a.queries = d_queries; a.Q = q; a.top_k = p->top_k; a.metric = L->metric;
        a.p = glide::BeamParamsHost{p->beam, p->max_iterations, p->min_iterations, p->hash_bit, p->hash_reset_interval};
        a.C = 1; a.out_ids = d_final_ids; a.out_dists = d_final_dists;
        a.segment_ids = L->d_routes; a.segment_num = S; a.parts = L->d_parts;
        a.ticket = ctx->ticket;
        cudaEvent_t k0, k1;
        LG_CUDA(ctx, cudaEventCreate(&k0));
        LG_CUDA(ctx, cudaEventCreate(&k1));
        LG_CUDA(ctx, cudaEventRecord(k0, ctx->stream));
        LG_CUDA(ctx, glide::launch_search(a, ctx->stream));
        LG_CUDA(ctx, cudaEventRecord(k1, ctx->stream));
        LG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        float ms = 0;
        cudaEventElapsedTime(&ms, k0, k1);
        cudaEventDestroy(k0);
        cudaEventDestroy(k1);
        L->last_stage_seconds[1] = ms / 1e3f;
        L->last_searched_partitions = (uint32_t) todo.size();
        ctx->last_ms = (L->last_stage_seconds[0] + L->last_stage_seconds[1]) * 1e3f;
        return GLIDE_OK;
    }
    if (max_stream_rows) {
        rc = ensure_slots(L, max_stream_rows, L->slot_has_knn, 64);
        if (rc) return rc;
    }
    // streamed partitions alternate between the two slots; uploads run ahead of the search kernels
    std::vector<uint32_t> streamed;
    for (uint32_t s : todo) if (!L->resident[s].rows) streamed.push_back(s);
    cudaEvent_t up_begin, up_end;
    LG_CUDA(ctx, cudaEventCreate(&up_begin));
    LG_CUDA(ctx, cudaEventCreate(&up_end));
    LG_CUDA(ctx, cudaEventRecord(up_begin, L->up));
    size_t next_upload = 0;
    auto upload = [&](size_t k) -> int {
        const uint32_t s = streamed[k];
        Slot &sl = L->slot[k & 1];
        LG_CUDA(ctx, cudaStreamWaitEvent(L->up, sl.computed, 0));   // the slot's previous partition has been searched
        int r = upload_rows(L, s, sl, L->up);
        if (r) return r;
        const uint32_t len = L->seg_len[s];
        LG_CUDA(ctx, cudaMemcpyAsync(sl.graph, L->h_graph + (size_t) L->seg_start[s] * L->degree, (size_t) len * L->degree * 4,
                                     cudaMemcpyHostToDevice, L->up));
        LG_CUDA(ctx, cudaMemcpyAsync(sl.map, L->h_map + L->seg_start[s], (size_t) len * 4, cudaMemcpyHostToDevice, L->up));
        LG_CUDA(ctx, cudaEventRecord(sl.uploaded, L->up));
        L->last_h2d_bytes += (double) len * (L->row_bytes() + L->degree * 4.0 + 4.0);
        L->last_uploaded_partitions++;
        return GLIDE_OK;
    };
    if (!streamed.empty()) {
        for (auto &sl : L->slot) LG_CUDA(ctx, cudaEventRecord(sl.computed, ctx->stream));
        rc = upload(next_upload++);
        if (rc) return rc;
    }
    size_t stream_k = 0;
    for (uint32_t s : todo) {
        const Slot *use = &L->resident[s];
        if (!use->rows) {
            Slot &sl = L->slot[stream_k & 1];
            if (next_upload < streamed.size()) { rc = upload(next_upload++); if (rc) return rc; }
            LG_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, sl.uploaded, 0));
            use = &sl;
        }
        rc = glide_search_on_sub(ctx, use->rows, L->dim, use->graph, L->degree, use->map, L->start_points[s], d_queries, q,
                                 L->d_routes, S, s, p, L->metric, d_final_ids, d_final_dists);
        if (rc) return rc;
        L->last_stage_seconds[1] += ctx->last_ms / 1e3f;
        L->last_searched_partitions++;
        if (!L->resident[s].rows) {
            LG_CUDA(ctx, cudaEventRecord(L->slot[stream_k & 1].computed, ctx->stream));
            stream_k++;
        }
    }
    float up_ms = 0;
    cudaEventRecord(up_end, L->up);
    cudaStreamSynchronize(L->up);
    cudaEventElapsedTime(&up_ms, up_begin, up_end);
    L->last_h2d_seconds = up_ms / 1e3;
    cudaEventDestroy(up_begin);
    cudaEventDestroy(up_end);
    ctx->last_ms = (L->last_stage_seconds[0] + L->last_stage_seconds[1]) * 1e3f;
    return GLIDE_OK;
}

// ---- merged index ------------------------------------------------------------------------------
// The reference declares GLIDE_large::build_with_merge (glide_large.cuh:96) and defines it nowhere;
// what follows is this library's own reading of "one graph over the whole set instead of a search
// per routed partition", made of the pieces the rest of the large path already has:
//   * every partition in one piece of device memory (needs all of them resident), its subgraph
//     rewritten from partition-local ids to reorder ids;
//   * links: a point whose list of partitions within boundary_factor of its nearest holds other
//     partitions than its own (select_segment_kernel's rule, the data points as queries) is searched
//     for in those partitions (the routed multi-partition search, results as reorder ids) and its
//     link_count nearest finds go into its row (link_merge_kernel);
//   * reverse edges over the whole graph, so that the neighbouring partition points back;
//   * search: the small path's kernel on that graph, entered at the nearest centroid's start point.
int glide_large_merge(glide_large *L, const float *d_centroids, uint32_t centroid_num, float boundary_factor, uint32_t link_count,
                      const glide_search_params *p_link, double *stats) {
    if (!L) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = L->ctx;
    const uint32_t S = (uint32_t) L->seg_len.size();
    if (!d_centroids || !p_link || centroid_num != S) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_merge: one centroid per partition expected");
    if (link_count < 1 || link_count > 32 || link_count >= L->degree || p_link->top_k != link_count)
        return fail(ctx, GLIDE_ERR_BAD_ARG, "large_merge: link_count must be in [1, 32], below the degree, and equal p_link->top_k");
    if (p_link->beam < 32 || p_link->beam % 32 || p_link->beam > 512 || p_link->top_k > p_link->beam)
        return fail(ctx, GLIDE_ERR_BAD_ARG, "large_merge: bad search parameters");
    uint64_t n64 = 0;
    for (uint32_t s = 0; s < S; s++) {
        if (L->seg_len[s] && !L->resident[s].rows) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_merge: every partition must be resident (glide_large_make_resident)");
        if (L->seg_start[s] != n64) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_merge: partitions must tile the rows in order");
        n64 += L->seg_len[s];
    }
    if (n64 == 0 || n64 >= 0xffffffffull) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_merge: empty or too large");
    const uint32_t n = (uint32_t) n64, dim = L->dim, degree = L->degree;
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    if (!L->arena_rows) {
        LG_CUDA(ctx, cudaMalloc(&L->arena_rows, (size_t) n * dim * 4));
        LG_CUDA(ctx, cudaMalloc(&L->merged_graph, (size_t) n * degree * 4));
        LG_CUDA(ctx, cudaMalloc(&L->arena_map, (size_t) n * 4));
        LG_CUDA(ctx, cudaMalloc(&L->d_gid, (size_t) n * 4));
        LG_CUDA(ctx, cudaMalloc(&L->d_start_global, (size_t) S * 4));
        LG_CUDA(ctx, cudaMalloc(&L->d_seg_start, (size_t) S * 4));
    }
    std::vector<uint32_t> start_global(S);
    for (uint32_t s = 0; s < S; s++) {
        start_global[s] = L->seg_start[s] + L->start_points[s];
        const uint32_t len = L->seg_len[s];
        if (len == 0) continue;
        const Slot &r = L->resident[s];
        const size_t lo = L->seg_start[s];
        if (!r.view) {
            LG_CUDA(ctx, cudaMemcpyAsync(L->arena_rows + lo * dim, r.rows, (size_t) len * dim * 4, cudaMemcpyDeviceToDevice, st));
            LG_CUDA(ctx, cudaMemcpyAsync(L->arena_map + lo, r.map, (size_t) len * 4, cudaMemcpyDeviceToDevice, st));
        }
        const size_t entries = (size_t) len * degree;
        globalise_kernel<<<(unsigned) ((entries + 255) / 256), 256, 0, st>>>(r.graph, entries, (uint32_t) lo, L->merged_graph + lo * degree);
    }
    LG_CUDA(ctx, cudaGetLastError());
    iota_kernel<<<(n + 255) / 256, 256, 0, st>>>(L->d_gid, n);
    LG_CUDA(ctx, cudaMemcpyAsync(L->d_start_global, start_global.data(), (size_t) S * 4, cudaMemcpyHostToDevice, st));
    LG_CUDA(ctx, cudaMemcpyAsync(L->d_seg_start, L->seg_start.data(), (size_t) S * 4, cudaMemcpyHostToDevice, st));
    // from here on the arena is the resident copy of rows and id maps: the per-partition copies go
    LG_CUDA(ctx, cudaStreamSynchronize(st));
    for (uint32_t s = 0; s < S; s++) {
        Slot &r = L->resident[s];
        if (L->seg_len[s] == 0 || r.view) continue;
        cudaFree(r.rows);
        cudaFree(r.map);
        r.rows = L->arena_rows + (size_t) L->seg_start[s] * dim;
        r.map = L->arena_map + L->seg_start[s];
        r.view = true;
    }
    // partition table of the link search: rows and local subgraph as they are resident, ids out as reorder ids
    std::vector<glide::PartitionRef> refs(S, glide::PartitionRef{nullptr, nullptr, nullptr, 0, 0});
    for (uint32_t s = 0; s < S; s++) {
        if (L->seg_len[s] == 0) continue;
        const Slot &r = L->resident[s];
        refs[s] = glide::PartitionRef{r.rows, r.graph, L->d_gid + L->seg_start[s], L->start_points[s], L->seg_len[s]};
    }
    LG_CUDA(ctx, cudaMemcpyAsync(L->d_parts, refs.data(), (size_t) S * sizeof(glide::PartitionRef), cudaMemcpyHostToDevice, st));
    LG_CUDA(ctx, cudaStreamSynchronize(st));   // start_global and refs are local vectors
    // links, a chunk of points at a time
    const uint32_t chunk = 1u << 18;
    const uint32_t rows_cap = n < chunk ? n : chunk;
    if ((size_t) rows_cap * S > L->routes_capacity) {
        if (L->d_routes) cudaFree(L->d_routes);
        L->d_routes = nullptr;
        LG_CUDA(ctx, cudaMalloc(&L->d_routes, (size_t) rows_cap * S * 4));
        L->routes_capacity = (size_t) rows_cap * S;
    }
    uint32_t *d_links = nullptr, *d_count = nullptr;
    float *d_link_d = nullptr;
    LG_CUDA(ctx, cudaMalloc(&d_links, (size_t) rows_cap * link_count * 4));
    LG_CUDA(ctx, cudaMalloc(&d_link_d, (size_t) rows_cap * link_count * 4));
    LG_CUDA(ctx, cudaMalloc(&d_count, 4));
    LG_CUDA(ctx, cudaMemsetAsync(d_count, 0, 4, st));
    std::vector<float> far((size_t) rows_cap * link_count, 3.402823466e+38f);
    cudaEvent_t e0, e1, e2;
    cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
    cudaEventRecord(e0, st);
    int rc = GLIDE_OK;
    for (uint32_t lo = 0; lo < n && rc == GLIDE_OK; lo += chunk) {
        const uint32_t cnt = n - lo < chunk ? n - lo : chunk;
        const float *d_points = L->arena_rows + (size_t) lo * dim;
        rc = glide_select_segments(ctx, d_points, cnt, dim, d_centroids, S, 1, boundary_factor, L->metric, L->d_routes);
        if (rc) break;
        drop_own_kernel<<<(cnt + 255) / 256, 256, 0, st>>>(L->d_routes, cnt, S, lo, L->d_seg_start);
        cudaMemsetAsync(d_links, 0xff, (size_t) cnt * link_count * 4, st);
        cudaMemcpyAsync(d_link_d, far.data(), (size_t) cnt * link_count * 4, cudaMemcpyHostToDevice, st);
        glide::SearchArgs a{};
        a.degree = degree; a.dim = dim; a.queries = d_points; a.Q = cnt; a.top_k = link_count; a.metric = L->metric;
        a.p = glide::BeamParamsHost{p_link->beam, p_link->max_iterations, p_link->min_iterations, p_link->hash_bit, p_link->hash_reset_interval};
        a.C = 1; a.out_ids = d_links; a.out_dists = d_link_d;
        a.segment_ids = L->d_routes; a.segment_num = S; a.parts = L->d_parts;
        a.ticket = ctx->ticket;
        cudaError_t ce = glide::launch_search(a, st);
        if (ce == cudaSuccess) {
            link_merge_kernel<<<(cnt + 255) / 256, 256, 0, st>>>(L->merged_graph + (size_t) lo * degree, d_links, cnt, degree, link_count, d_count);
            ce = cudaGetLastError();
        }
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
        if (ce != cudaSuccess) rc = fail(ctx, GLIDE_ERR_CUDA, "large_merge: %s", cudaGetErrorString(ce));
    }
    cudaEventRecord(e1, st);
    uint32_t with_links = 0;
    if (rc == GLIDE_OK && cudaMemcpy(&with_links, d_count, 4, cudaMemcpyDeviceToHost) != cudaSuccess) rc = fail(ctx, GLIDE_ERR_CUDA, "large_merge: copy failed");
    cudaFree(d_links); cudaFree(d_link_d); cudaFree(d_count);
    if (rc == GLIDE_OK) rc = glide_reverse_graph(ctx, L->merged_graph, n, degree);
    cudaEventRecord(e2, st);
    cudaEventSynchronize(e2);
    float ms_links = 0, ms_rev = 0;
    cudaEventElapsedTime(&ms_links, e0, e1);
    cudaEventElapsedTime(&ms_rev, e1, e2);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    if (stats) { stats[0] = ms_links / 1e3; stats[1] = ms_rev / 1e3; stats[2] = with_links; }
    return rc;
}

// One beam search per query over the merged graph, entered at the nearest centroid's start point
// (glide_search on the arena); ids come back as original ids.
int glide_large_search_merged(glide_large *L, const float *d_queries, uint32_t q, const float *d_centroids, uint32_t centroid_num,
                              const glide_search_params *p, uint32_t *d_out_ids, float *d_out_dists) {
    if (!L) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = L->ctx;
    if (!L->merged_graph) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_search_merged: no merged index (glide_large_merge)");
    const uint32_t S = (uint32_t) L->seg_len.size();
    if (centroid_num != S) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_search_merged: one centroid per partition expected");
    const uint32_t n = L->seg_start[S - 1] + L->seg_len[S - 1];
    int rc = glide_search(ctx, L->arena_rows, n, L->dim, L->merged_graph, L->degree, d_centroids, S, L->d_start_global, d_queries, q, p,
                          L->metric, d_out_ids, d_out_dists);
    if (rc || q == 0) return rc;
    const size_t count = (size_t) q * p->top_k;
    map_ids_kernel<<<(unsigned) ((count + 255) / 256), 256, 0, ctx->stream>>>(d_out_ids, L->arena_map, count);
    LG_CUDA(ctx, cudaGetLastError());
    LG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return GLIDE_OK;
}

// The merged graph (rows x degree, reorder ids) into host memory, for files and tests.
int glide_large_merged_graph(const glide_large *L, uint32_t *h_out) {
    if (!L || !h_out) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = L->ctx;
    if (!L->merged_graph) return fail(ctx, GLIDE_ERR_BAD_ARG, "large_merged_graph: no merged index (glide_large_merge)");
    const uint32_t S = (uint32_t) L->seg_len.size();
    const size_t n = (size_t) L->seg_start[S - 1] + L->seg_len[S - 1];
    LG_CUDA(ctx, cudaSetDevice(ctx->device));
    LG_CUDA(ctx, cudaMemcpy(h_out, L->merged_graph, n * L->degree * 4, cudaMemcpyDeviceToHost));
    return GLIDE_OK;
}

}  // extern "C"
