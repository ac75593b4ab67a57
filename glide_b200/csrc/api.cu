// C ABI (include/glide_b200.h): argument checks, scratch memory, stream and timing around
// the kernel launchers. No compute happens on the host; there is no CPU fallback.
#include <algorithm>
#include <atomic>
#include <cfloat>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/glide_b200.h"
#include "ctx.h"
#include "kernels.h"
#include "scan.cuh"

using namespace glide;

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

#define GL_CUDA(ctx, call)                                                                          \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess)                                                                      \
            return fail(ctx, e_ == cudaErrorMemoryAllocation ? GLIDE_ERR_NO_MEMORY : GLIDE_ERR_CUDA, \
                        "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__);       \
    } while (0)

#define GL_REQUIRE(ctx, cond, code, msg)               \
    do {                                                \
        if (!(cond)) return fail(ctx, code, "%s", msg); \
    } while (0)

size_t align256(size_t x) { return (x + 255) & ~(size_t) 255; }

int ensure_ws(glide_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->ws_bytes) return GLIDE_OK;
    if (ctx->ws) {
        GL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        GL_CUDA(ctx, cudaFree(ctx->ws));
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
    }
    GL_CUDA(ctx, cudaMalloc(&ctx->ws, bytes));
    ctx->ws_bytes = bytes;
    return GLIDE_OK;
}

struct Bump {
    char *base;
    size_t off = 0;
    explicit Bump(void *b) : base(static_cast<char *>(b)) {}
    template<typename T>
    T *take(size_t count) {
        T *p = reinterpret_cast<T *>(base + off);
        off += align256(count * sizeof(T));
        return p;
    }
};

int check_params(glide_ctx *ctx, const glide_search_params *p, uint32_t degree) {
    GL_REQUIRE(ctx, p != nullptr, GLIDE_ERR_BAD_ARG, "search params are null");
    GL_REQUIRE(ctx, p->beam >= 32 && p->beam % 32 == 0, GLIDE_ERR_BAD_ARG, "beam must be a positive multiple of 32");
    GL_REQUIRE(ctx, p->beam <= 512, GLIDE_ERR_UNSUPPORTED, "Unsupported beam");               // kernel_config.cuh:47-48
    GL_REQUIRE(ctx, degree >= 1 && degree <= 256, GLIDE_ERR_UNSUPPORTED, "Unsupported graph_degree");  // :59-60
    GL_REQUIRE(ctx, p->max_iterations >= 1, GLIDE_ERR_BAD_ARG, "max_iterations must be >= 1");
    GL_REQUIRE(ctx, p->hash_bit >= 4 && p->hash_bit <= 13, GLIDE_ERR_BAD_ARG, "hash_bit out of range");
    GL_REQUIRE(ctx, p->hash_reset_interval >= 1, GLIDE_ERR_BAD_ARG, "hash_reset_interval must be >= 1");
    return GLIDE_OK;
}

BeamParamsHost to_host(const glide_search_params *p) {
    return BeamParamsHost{p->beam, p->max_iterations, p->min_iterations, p->hash_bit, p->hash_reset_interval};
}

struct Timed {
    glide_ctx *ctx;
    explicit Timed(glide_ctx *c) : ctx(c) { cudaEventRecord(ctx->ev_start, ctx->stream); }
    int finish() {
        cudaEventRecord(ctx->ev_stop, ctx->stream);
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return fail(ctx, GLIDE_ERR_CUDA, "kernel execution failed: %s", cudaGetErrorString(e));
        cudaEventElapsedTime(&ctx->last_ms, ctx->ev_start, ctx->ev_stop);
        return GLIDE_OK;
    }
};

unsigned long long *counters_or_null(glide_ctx *ctx) {
    if (!ctx->counters_on) return nullptr;
    cudaMemsetAsync(ctx->counters, 0, 4 * sizeof(unsigned long long), ctx->stream);
    return ctx->counters;
}

uint64_t splitmix64(uint64_t &x) {
    uint64_t z = (x += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

uint64_t gcd64(uint64_t a, uint64_t b) {
    while (b) { const uint64_t t = a % b; a = b; b = t; }
    return a;
}

}  // namespace

extern "C" {

static int build_nnd_simt(glide_ctx *ctx, const float *d_reorder_data, uint32_t rows, uint32_t dim,
                          const uint32_t *h_segment_start, const uint32_t *h_segment_length, uint32_t S, uint32_t knn_degree,
                          uint32_t K, uint32_t max_iterations, float termination_threshold, uint32_t sample,
                          uint32_t exact_max_rows, uint64_t seed, int metric, uint32_t row_base, int32_t *d_knn,
                          uint32_t *iterations_run, bool skip_exact);

int glide_ctx_create(int device, glide_ctx **out) {
    if (!out) return GLIDE_ERR_BAD_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) return GLIDE_ERR_CUDA;
    glide_ctx *ctx = new (std::nothrow) glide_ctx();
    if (!ctx) return GLIDE_ERR_NO_MEMORY;
    ctx->device = device;
    if (cudaSetDevice(device) != cudaSuccess || cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreate(&ctx->ev_start) != cudaSuccess || cudaEventCreate(&ctx->ev_stop) != cudaSuccess ||
        cudaEventCreate(&ctx->ev_mid) != cudaSuccess ||
        cudaMalloc(&ctx->counters, 4 * sizeof(unsigned long long)) != cudaSuccess ||
        cudaMalloc(&ctx->tc_norms, (4096 + 128 + 1) * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&ctx->ticket, 2 * sizeof(uint32_t)) != cudaSuccess) {
        delete ctx;
        return GLIDE_ERR_CUDA;
    }
    ctx->start_point_word = ctx->ticket + 1;
    // load the common kernel instances and let the driver size its local-memory reservation now,
    // not inside the first timed stage
    if (preload_build_kernels(ctx->stream) != cudaSuccess || preload_search_kernels(ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
        glide_ctx_destroy(ctx);
        return GLIDE_ERR_CUDA;
    }
    *out = ctx;
    return GLIDE_OK;
}

void glide_ctx_destroy(glide_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    glide_comm_release(ctx);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->tc_norms) cudaFree(ctx->tc_norms);
    if (ctx->ticket) cudaFree(ctx->ticket);
    if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
    if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
    if (ctx->ev_mid) cudaEventDestroy(ctx->ev_mid);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *glide_last_error(const glide_ctx *ctx) { return ctx ? ctx->error.c_str() : "null context"; }
void *glide_ctx_stream(glide_ctx *ctx) { return ctx ? (void *) ctx->stream : nullptr; }
float glide_last_kernel_ms(const glide_ctx *ctx) { return ctx ? ctx->last_ms : 0.0f; }
size_t glide_ctx_workspace_bytes(const glide_ctx *ctx) { return ctx ? ctx->ws_bytes : 0; }

void glide_last_search_split_ms(const glide_ctx *ctx, float out[2]) {
    if (!ctx || !out) return;
    out[0] = ctx->split_ms[0];
    out[1] = ctx->split_ms[1];
}

uint32_t glide_last_search_launches(const glide_ctx *ctx) { return ctx ? ctx->last_launches : 0; }

void glide_enable_counters(glide_ctx *ctx, int on) { if (ctx) ctx->counters_on = on != 0; }

int glide_read_counters(glide_ctx *ctx, uint64_t out[4]) {
    if (!ctx || !out) return GLIDE_ERR_BAD_ARG;
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    GL_CUDA(ctx, cudaMemcpyAsync(out, ctx->counters, 4 * sizeof(uint64_t), cudaMemcpyDeviceToHost, ctx->stream));
    GL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return GLIDE_OK;
}

// params.cuh:49-66
uint32_t glide_calculate_hash_bitlen(uint32_t beam, uint32_t graph_degree, float max_fill_rate, uint32_t min_bitlen) {
    const uint32_t max_visited = beam + graph_degree;
    uint32_t lo = 8;
    const uint32_t hi = 13;
    if (lo < min_bitlen) lo = min_bitlen;
    uint32_t bitlen = lo;
    while (max_visited > (float) (1u << bitlen) * max_fill_rate) bitlen += 1;
    if (bitlen > hi) bitlen = hi;
    return bitlen;
}

// params.cuh:68-80
uint32_t glide_calculate_hash_reset_interval(uint32_t beam, uint32_t graph_degree, float max_fill_rate,
                                             uint32_t hash_bitlen) {
    uint32_t interval = 1;
    while (true) {
        const uint32_t max_visited = beam + graph_degree * (interval + 1);
        if (max_visited > (float) (1u << hash_bitlen) * max_fill_rate) break;
        interval += 1;
    }
    return interval;
}

// params.cuh:82-99
void glide_adjust_search_params(uint32_t min_iterations, uint32_t *max_iterations, uint32_t *beam) {
    uint32_t m = *max_iterations;
    if (*max_iterations == 0) m = (uint32_t) (1 + std::min(*beam * 1.1, *beam + 10.0));
    if (*max_iterations < min_iterations) m = min_iterations;
    if (*max_iterations < m) *max_iterations = m;
    if (*beam % 32) *beam += 32 - (*beam % 32);
}

// ---- memory helpers ----------------------------------------------------------------------
int glide_malloc(glide_ctx *ctx, size_t bytes, void **d_out) {
    if (!ctx || !d_out) return GLIDE_ERR_BAD_ARG;
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    GL_CUDA(ctx, cudaMalloc(d_out, bytes ? bytes : 1));
    return GLIDE_OK;
}
void glide_free(void *device_ptr) { if (device_ptr) cudaFree(device_ptr); }
int glide_memcpy_h2d(glide_ctx *ctx, void *d_dst, const void *h_src, size_t bytes) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    GL_CUDA(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return GLIDE_OK;
}
int glide_memcpy_d2h(glide_ctx *ctx, void *h_dst, const void *d_src, size_t bytes) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    GL_CUDA(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    GL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return GLIDE_OK;
}
int glide_memset_u32(glide_ctx *ctx, uint32_t *d_dst, uint32_t value, size_t count) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    const uint8_t b = value & 0xff;
    if (((value >> 8) & 0xff) == b && ((value >> 16) & 0xff) == b && (value >> 24) == b) {
        GL_CUDA(ctx, cudaMemsetAsync(d_dst, b, count * 4, ctx->stream));
    } else {
        std::vector<uint32_t> h(count, value);
        GL_CUDA(ctx, cudaMemcpyAsync(d_dst, h.data(), count * 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    GL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return GLIDE_OK;
}

// ---- partition ---------------------------------------------------------------------------
int glide_kmeans_fit(glide_ctx *ctx, const float *d_sample, uint32_t n, uint32_t dim, uint32_t C, uint32_t max_iter,
                     int metric, int init, float *d_centroids, uint32_t *d_labels_or_null, uint32_t *iterations_run) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_sample && d_centroids && dim > 0, GLIDE_ERR_BAD_ARG, "kmeans: null pointer or zero dim");
    GL_REQUIRE(ctx, C >= 1 && n >= C, GLIDE_ERR_BAD_ARG, "kmeans: fewer rows than centroids");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroids_num");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    if (max_iter == 0) max_iter = 25;
    const size_t need = 4 * align256((size_t) n * 4) + align256(slot_scratch_words(n, C) * 4) +
                        3 * align256((size_t) (C + 2) * 4) + align256(scan_tmp_bytes(C + 1)) + 256 +
                        align256(farthest_first_scratch_bytes(n));
    int rc = ensure_ws(ctx, need);
    if (rc) return rc;
    Bump b(ctx->ws);
    uint32_t *labels_a = b.take<uint32_t>(n), *labels_b = b.take<uint32_t>(n);
    uint32_t *slot = b.take<uint32_t>(n), *members = b.take<uint32_t>(n);
    uint32_t *hist = b.take<uint32_t>(slot_scratch_words(n, C));
    uint32_t *cnt = b.take<uint32_t>(C + 2), *off = b.take<uint32_t>(C + 2), *changed = b.take<uint32_t>(C + 2);
    void *scan_tmp = b.take<char>(scan_tmp_bytes(C + 1));
    void *ff_tmp = b.take<char>(farthest_first_scratch_bytes(n));
    cudaStream_t st = ctx->stream;
    Timed timer(ctx);
    if (init == 0) {
        GL_CUDA(ctx, cudaMemcpyAsync(d_centroids, d_sample, (size_t) C * dim * 4, cudaMemcpyDeviceToDevice, st));
    } else {
        GL_CUDA(ctx, launch_farthest_first(d_sample, n, dim, C, d_centroids, ff_tmp, st));
    }
    GL_CUDA(ctx, cudaMemsetAsync(labels_b, 0xff, (size_t) n * 4, st));
    uint32_t rounds = 0;
    uint32_t *cur = labels_a, *prev = labels_b;
    for (uint32_t it = 0; it < max_iter; it++) {
        AssignArgs a{d_sample, n, dim, d_centroids, C, -1.0f, metric, cur, nullptr, C <= 4096 ? ctx->tc_norms : nullptr, nullptr};
        GL_CUDA(ctx, launch_assign(a, st));
        GL_CUDA(ctx, launch_count_changed(cur, prev, n, changed, st));
        uint32_t h_changed = 0;
        GL_CUDA(ctx, cudaMemcpyAsync(&h_changed, changed, 4, cudaMemcpyDeviceToHost, st));
        GL_CUDA(ctx, cudaStreamSynchronize(st));
        rounds++;
        std::swap(cur, prev);  // prev now holds the latest labels
        if (h_changed == 0) break;
        GL_CUDA(ctx, launch_slots(prev, n, C, slot, cnt, hist, st));
        GL_CUDA(ctx, exclusive_scan_u32(cnt, C, off, scan_tmp, st));
        GL_CUDA(ctx, launch_scatter_members(prev, slot, off, n, members, st));
        GL_CUDA(ctx, launch_centroid_update(d_sample, dim, members, off, cnt, C, d_centroids, st));
    }
    if (d_labels_or_null) GL_CUDA(ctx, cudaMemcpyAsync(d_labels_or_null, prev, (size_t) n * 4, cudaMemcpyDeviceToDevice, st));
    if (iterations_run) *iterations_run = rounds;
    return timer.finish();
}

// Sample ids: an arithmetic progression modulo n with a seeded stride coprime to n, i.e.
// floor(n*sample_factor) distinct rows spread over the whole set. (The reference shuffles
// all ids with an unseeded generator and takes the first ones, partition.cuh:25-31.)
static void sample_ids(uint32_t n, uint32_t sample_num, uint64_t seed, std::vector<uint32_t> &ids) {
    uint64_t s = seed;
    uint64_t stride = splitmix64(s) % n;
    if (stride == 0) stride = 1;
    while (gcd64(stride, n) != 1) stride = stride % n + 1;
    const uint64_t offset = splitmix64(s) % n;
    ids.resize(sample_num);
    for (uint32_t i = 0; i < sample_num; i++) ids[i] = (uint32_t) ((offset + (uint64_t) i * stride) % n);
}

int glide_sample_ids(uint32_t n, uint32_t sample_num, uint64_t seed, uint32_t *h_out) {
    if (!h_out || n == 0 || sample_num > n) return GLIDE_ERR_BAD_ARG;
    std::vector<uint32_t> ids;
    sample_ids(n, sample_num, seed, ids);
    std::memcpy(h_out, ids.data(), (size_t) sample_num * 4);
    return GLIDE_OK;
}

int glide_get_centroids(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, uint32_t C, float sample_factor,
                        uint64_t seed, uint32_t max_iter, int metric, float *d_centroids, uint32_t *iterations_run) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_data && d_centroids && n > 0 && dim > 0, GLIDE_ERR_BAD_ARG, "get_centroids: bad argument");
    const uint32_t sample_num = (uint32_t) ((double) n * sample_factor);  // partition.cuh:17
    GL_REQUIRE(ctx, sample_num >= C && sample_num <= n, GLIDE_ERR_BAD_ARG,
               "get_centroids: sample smaller than centroid_num (raise sample_factor)");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    std::vector<uint32_t> ids;
    sample_ids(n, sample_num, seed, ids);
    float *d_sample = nullptr;
    uint32_t *d_ids = nullptr;
    GL_CUDA(ctx, cudaMalloc(&d_sample, (size_t) sample_num * dim * 4));
    cudaError_t e = cudaMalloc(&d_ids, (size_t) sample_num * 4);
    if (e != cudaSuccess) { cudaFree(d_sample); return fail(ctx, GLIDE_ERR_NO_MEMORY, "cudaMalloc failed"); }
    int rc = GLIDE_OK;
    e = cudaMemcpyAsync(d_ids, ids.data(), (size_t) sample_num * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = launch_gather_rows(d_data, d_ids, sample_num, dim, d_sample, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) rc = fail(ctx, GLIDE_ERR_CUDA, "sample gather failed: %s", cudaGetErrorString(e));
    if (rc == GLIDE_OK) rc = glide_kmeans_fit(ctx, d_sample, sample_num, dim, C, max_iter, metric, 1, d_centroids, nullptr, iterations_run);
    cudaFree(d_sample);
    cudaFree(d_ids);
    return rc;
}

int glide_define_partition(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, const float *d_centroids,
                           uint32_t C, float boundary_factor, int metric, uint32_t *d_segment_index,
                           uint32_t *h_segment_start, uint32_t *h_segment_length) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_data && d_centroids && d_segment_index && h_segment_start && h_segment_length, GLIDE_ERR_BAD_ARG,
               "define_partition: null pointer");
    GL_REQUIRE(ctx, n > 0 && dim > 0 && C >= 1, GLIDE_ERR_BAD_ARG, "define_partition: zero size");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroids_num");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t need = 4 * align256((size_t) n * 4) + align256(slot_scratch_words(n, C) * 4) + align256((size_t) (C + 1) * 4) + 256;
    int rc = ensure_ws(ctx, need);
    if (rc) return rc;
    Bump b(ctx->ws);
    uint32_t *nearest = b.take<uint32_t>(n), *bkey = b.take<uint32_t>(n), *slot = b.take<uint32_t>(n), *bslot = b.take<uint32_t>(n);
    uint32_t *hist = b.take<uint32_t>(slot_scratch_words(n, C));
    uint32_t *totals = b.take<uint32_t>(C + 1);
    cudaStream_t st = ctx->stream;
    Timed timer(ctx);
    unsigned long long *cnt = counters_or_null(ctx);
    AssignArgs a{d_data, n, dim, d_centroids, C, boundary_factor, metric, nearest, bkey, ctx->tc_norms, cnt ? cnt + 3 : nullptr};
    GL_CUDA(ctx, launch_assign(a, st));
    GL_CUDA(ctx, launch_slots(nearest, n, C, slot, totals, hist, st));
    GL_CUDA(ctx, launch_slots(bkey, n, 1, bslot, totals + C, hist, st));
    GL_CUDA(ctx, launch_pack_seg_index(nearest, slot, bslot, n, d_segment_index, st));
    GL_CUDA(ctx, cudaMemcpyAsync(h_segment_length, totals, (size_t) (C + 1) * 4, cudaMemcpyDeviceToHost, st));
    rc = timer.finish();
    if (rc) return rc;
    uint32_t start = 0;  // partition.cuh:111-115
    for (uint32_t i = 0; i <= C; i++) {
        h_segment_start[i] = start;
        start += h_segment_length[i];
    }
    return GLIDE_OK;
}

int glide_reorder(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, const uint32_t *d_segment_index,
                  const uint32_t *h_segment_start, uint32_t C, float *d_reorder_data, uint32_t *d_map) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_data && d_segment_index && h_segment_start && d_reorder_data && d_map, GLIDE_ERR_BAD_ARG,
               "reorder: null pointer");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    int rc = ensure_ws(ctx, align256((size_t) (C + 1) * 4));
    if (rc) return rc;
    uint32_t *d_start = static_cast<uint32_t *>(ctx->ws);
    Timed timer(ctx);
    GL_CUDA(ctx, cudaMemcpyAsync(d_start, h_segment_start, (size_t) (C + 1) * 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, launch_reorder(d_data, n, dim, d_segment_index, d_start, d_reorder_data, d_map, ctx->stream));
    return timer.finish();
}

int glide_preprocess(glide_ctx *ctx, const float *d_data, uint32_t n, uint32_t dim, uint32_t C, float boundary_factor,
                     float sample_factor, int metric, uint64_t seed, float *d_centroids, uint32_t *h_segment_start,
                     uint32_t *h_segment_length, float **d_reorder_data_out, uint32_t **d_map_out,
                     uint32_t *reorder_num_out) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_reorder_data_out && d_map_out && reorder_num_out, GLIDE_ERR_BAD_ARG, "preprocess: null output");
    *d_reorder_data_out = nullptr;
    *d_map_out = nullptr;
    float total_ms = 0.0f;
    int rc = glide_get_centroids(ctx, d_data, n, dim, C, sample_factor, seed, 0, metric, d_centroids, nullptr);
    if (rc) return rc;
    total_ms += ctx->last_ms;
    uint32_t *d_seg_index = nullptr;
    GL_CUDA(ctx, cudaMalloc(&d_seg_index, (size_t) n * 3 * 4));
    rc = glide_define_partition(ctx, d_data, n, dim, d_centroids, C, boundary_factor, metric, d_seg_index,
                                h_segment_start, h_segment_length);
    total_ms += ctx->last_ms;
    if (rc) { cudaFree(d_seg_index); return rc; }
    const uint32_t reorder_num = n + h_segment_length[C];  // partition.cuh:182
    float *d_reorder = nullptr;
    uint32_t *d_map = nullptr;
    cudaError_t e = cudaMalloc(&d_reorder, (size_t) reorder_num * dim * 4);
    if (e == cudaSuccess) e = cudaMalloc(&d_map, (size_t) reorder_num * 4);
    if (e != cudaSuccess) {
        cudaFree(d_seg_index); cudaFree(d_reorder);
        return fail(ctx, GLIDE_ERR_NO_MEMORY, "preprocess: cudaMalloc failed: %s", cudaGetErrorString(e));
    }
    rc = glide_reorder(ctx, d_data, n, dim, d_seg_index, h_segment_start, C, d_reorder, d_map);
    total_ms += ctx->last_ms;
    cudaFree(d_seg_index);
    if (rc) { cudaFree(d_reorder); cudaFree(d_map); return rc; }
    *d_reorder_data_out = d_reorder;
    *d_map_out = d_map;
    *reorder_num_out = reorder_num;
    ctx->last_ms = total_ms;
    return GLIDE_OK;
}

// ---- kNN -----------------------------------------------------------------------------------
int glide_build_nnd(glide_ctx *ctx, const float *d_reorder_data, uint32_t rows, uint32_t dim,
                    const uint32_t *h_segment_start, const uint32_t *h_segment_length, uint32_t S, uint32_t knn_degree,
                    uint32_t max_iterations, float termination_threshold, uint32_t sample, uint32_t exact_max_rows,
                    uint64_t seed, int metric, int32_t *d_knn, uint32_t *iterations_run) {
    return glide_build_nnd_range(ctx, d_reorder_data, rows, dim, h_segment_start, h_segment_length, S, knn_degree,
                                 max_iterations, termination_threshold, sample, exact_max_rows, seed, metric, 0, d_knn,
                                 iterations_run);
}

int glide_build_nnd_range(glide_ctx *ctx, const float *d_reorder_data, uint32_t rows, uint32_t dim,
                          const uint32_t *h_segment_start, const uint32_t *h_segment_length, uint32_t S,
                          uint32_t knn_degree, uint32_t max_iterations, float termination_threshold, uint32_t sample,
                          uint32_t exact_max_rows, uint64_t seed, int metric, uint32_t row_base, int32_t *d_knn,
                          uint32_t *iterations_run) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_reorder_data && h_segment_start && h_segment_length && d_knn, GLIDE_ERR_BAD_ARG, "build_nnd: null pointer");
    GL_REQUIRE(ctx, rows > 0 && dim > 0 && S >= 1, GLIDE_ERR_BAD_ARG, "build_nnd: zero size");
    GL_REQUIRE(ctx, knn_degree >= 1 && knn_degree <= 64, GLIDE_ERR_UNSUPPORTED, "build_nnd: knn_degree must be <= 64");
    if (max_iterations == 0) max_iterations = 20;              // params.cuh:20
    if (termination_threshold < 0) termination_threshold = 1e-4f;  // params.cuh:21
    if (sample == 0) sample = 32;
    GL_REQUIRE(ctx, sample <= 32, GLIDE_ERR_UNSUPPORTED, "build_nnd: sample must be <= 32");
    uint64_t covered = 0;
    for (uint32_t s = 0; s < S; s++) {
        GL_REQUIRE(ctx, h_segment_start[s] == covered, GLIDE_ERR_BAD_ARG, "build_nnd: segments must tile the rows in order");
        covered += h_segment_length[s];
    }
    GL_REQUIRE(ctx, covered == rows, GLIDE_ERR_BAD_ARG, "build_nnd: segment lengths do not sum to the row count");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    const uint32_t K = knn_degree <= 32 ? 32 : 64;
    // Partitions of at most exact_max_rows rows get their exact kNN rows from an all-pairs kernel,
    // larger ones run NN-descent. Where the tensor-core kernel serves the shape, all pairs stay
    // cheaper than descent up to about a million rows per partition (4 x 10^12 pair distances per
    // second against ~1.3 x 10^6 rows per second of descent); the fp32 register-tile kernel gives way
    // at 16,384.
    const bool tc = knn_tc_eligible(d_reorder_data, dim, knn_degree);
    if (exact_max_rows == 0xffffffffu) exact_max_rows = tc ? (1u << 20) : 16384;
    if (tc) {
        bool any = false;
        for (uint32_t s = 0; s < S; s++) any = any || (h_segment_length[s] >= 1 && h_segment_length[s] <= exact_max_rows);
        if (any) {
            int rc0 = ensure_ws(ctx, knn_tc_scratch_bytes(rows, knn_degree));
            if (rc0) return rc0;
            Timed timer0(ctx);
            uint32_t failed = 0;
            cudaError_t e0 = launch_knn_tc(d_reorder_data, rows, dim, h_segment_start, h_segment_length, S, exact_max_rows,
                                           knn_degree, row_base, ctx->ws, d_knn, &failed, ctx->stream);
            if (e0 != cudaSuccess && e0 != cudaErrorNotSupported)
                return fail(ctx, GLIDE_ERR_CUDA, "tensor-core kNN: %s", cudaGetErrorString(e0));
            rc0 = timer0.finish();
            if (rc0) return rc0;
            if (e0 == cudaSuccess && !failed) {
                bool rest = false;   // partitions beyond exact_max_rows are left for NN-descent below
                for (uint32_t s = 0; s < S; s++) rest = rest || h_segment_length[s] > exact_max_rows;
                if (iterations_run) *iterations_run = 0;
                if (!rest) return GLIDE_OK;
                const float tc_ms = ctx->last_ms;
                rc0 = build_nnd_simt(ctx, d_reorder_data, rows, dim, h_segment_start, h_segment_length, S, knn_degree, K,
                                     max_iterations, termination_threshold, sample, exact_max_rows, seed, metric, row_base,
                                     d_knn, iterations_run, /*skip_exact=*/true);
                ctx->last_ms += tc_ms;
                return rc0;
            }
            // no tensor map, a wait that ran out, or a candidate buffer that overflowed: the fp32
            // kernels redo everything; the time of the attempt stays in the stage's time
            if (exact_max_rows > 16384) exact_max_rows = 16384;
            const float tc_ms = ctx->last_ms;
            rc0 = build_nnd_simt(ctx, d_reorder_data, rows, dim, h_segment_start, h_segment_length, S, knn_degree, K,
                                 max_iterations, termination_threshold, sample, exact_max_rows, seed, metric, row_base, d_knn,
                                 iterations_run, false);
            ctx->last_ms += tc_ms;
            ctx->tc_knn_fallbacks++;
            return rc0;
        }
    }
    return build_nnd_simt(ctx, d_reorder_data, rows, dim, h_segment_start, h_segment_length, S, knn_degree, K, max_iterations,
                          termination_threshold, sample, exact_max_rows, seed, metric, row_base, d_knn, iterations_run, false);
}

uint32_t glide_tc_knn_fallbacks(const glide_ctx *ctx) { return ctx ? ctx->tc_knn_fallbacks : 0; }

// The fp32 kernels of the kNN stage: the register-tile all-pairs kernel for partitions of at most
// exact_max_rows rows (unless skip_exact: the tensor-core kernel has done them) and NN-descent for the rest.
static int build_nnd_simt(glide_ctx *ctx, const float *d_reorder_data, uint32_t rows, uint32_t dim,
                          const uint32_t *h_segment_start, const uint32_t *h_segment_length, uint32_t S, uint32_t knn_degree,
                          uint32_t K, uint32_t max_iterations, float termination_threshold, uint32_t sample,
                          uint32_t exact_max_rows, uint64_t seed, int metric, uint32_t row_base, int32_t *d_knn,
                          uint32_t *iterations_run, bool skip_exact) {
    const uint32_t tile_count = skip_exact ? 0 : segment_knn_tile_count(h_segment_length, S, exact_max_rows);
    bool need_nnd = false;
    for (uint32_t s = 0; s < S; s++) need_nnd = need_nnd || h_segment_length[s] > exact_max_rows;
    const size_t nnd_bytes = need_nnd ? nnd_workspace_bytes(rows, K, sample, S) : 0;
    int rc = ensure_ws(ctx, nnd_bytes + 2 * align256((size_t) S * 4) + align256((size_t) tile_count * 12) + 256);
    if (rc) return rc;
    Bump b(ctx->ws);
    uint32_t *d_start = b.take<uint32_t>(S), *d_len = b.take<uint32_t>(S);
    uint32_t *d_tiles = b.take<uint32_t>((size_t) tile_count * 3 + 1);
    void *work = b.take<char>(nnd_bytes);
    std::vector<uint32_t> h_tiles((size_t) tile_count * 3 + 1);
    if (tile_count) segment_knn_fill_tiles(h_segment_start, h_segment_length, S, exact_max_rows, h_tiles.data());
    // empty segments (C == 1 leaves the boundary segment empty, partition_kernel.cuh:58) need no launch
    Timed timer(ctx);
    GL_CUDA(ctx, cudaMemcpyAsync(d_start, h_segment_start, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaMemcpyAsync(d_len, h_segment_length, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (iterations_run) *iterations_run = 0;
    if (tile_count) {
        GL_CUDA(ctx, cudaMemcpyAsync(d_tiles, h_tiles.data(), (size_t) tile_count * 12, cudaMemcpyHostToDevice, ctx->stream));
        GL_CUDA(ctx, launch_segment_knn(d_reorder_data, dim, d_tiles, tile_count, knn_degree, row_base, d_knn, ctx->stream));
    }
    if (!need_nnd) return timer.finish();
    NndArgs a{};
    a.data = d_reorder_data; a.rows = rows; a.dim = dim;
    a.seg_start = d_start; a.seg_len = d_len; a.S = S; a.min_seg_len = exact_max_rows + 1;
    a.K = K; a.sample = sample; a.max_iterations = max_iterations; a.termination_threshold = termination_threshold;
    a.seed = seed; a.metric = metric; a.workspace = work; a.workspace_bytes = nnd_bytes; a.row_base = row_base;
    a.out_knn = d_knn; a.out_degree = knn_degree; a.iterations_run = iterations_run; a.stage_ms = nullptr;
    GL_CUDA(ctx, run_nn_descent(a, ctx->stream));
    return timer.finish();
}

int glide_bruteforce_knn(glide_ctx *ctx, const float *d_base, uint32_t n, const float *d_queries, uint32_t q,
                         uint32_t dim, uint32_t k, int metric, uint32_t *d_out_ids, float *d_out_dists) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_base && d_queries && d_out_ids, GLIDE_ERR_BAD_ARG, "bruteforce_knn: null pointer");
    GL_REQUIRE(ctx, n > 0 && dim > 0, GLIDE_ERR_BAD_ARG, "bruteforce_knn: zero size");
    GL_REQUIRE(ctx, k >= 1 && k <= 128 && k <= n, GLIDE_ERR_UNSUPPORTED, "bruteforce_knn: k must be in [1, min(128, n)]");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    const uint32_t splits = bruteforce_default_splits(n, q);
    int rc = ensure_ws(ctx, bruteforce_scratch_bytes(q, k, splits) + 256);
    if (rc) return rc;
    Timed timer(ctx);
    GL_CUDA(ctx, launch_bruteforce(d_base, n, d_queries, q, dim, k, metric, splits, ctx->ws, d_out_ids, d_out_dists, ctx->stream));
    return timer.finish();
}

// ---- graph build ---------------------------------------------------------------------------
int glide_start_point_select(const uint32_t *h_segment_start, const uint32_t *h_segment_length, uint32_t S,
                             const uint32_t *h_map, uint64_t seed, uint32_t *h_local, uint32_t *h_original) {
    if (!h_segment_start || !h_segment_length || !h_local) return GLIDE_ERR_BAD_ARG;
    uint64_t s = seed;
    for (uint32_t i = 0; i < S; i++) {  // glide_impl.cuh:59-68
        const uint32_t len = h_segment_length[i];
        const uint32_t id = len ? (uint32_t) (splitmix64(s) % len) : 0;  // an empty segment (C == 1) gets 0
        h_local[i] = id;
        if (i + 1 != S && h_original && h_map) h_original[i] = h_map[h_segment_start[i] + id];
    }
    return GLIDE_OK;
}

static uint32_t longest_partition(const uint32_t *h_len, uint32_t lo, uint32_t hi) {
    uint32_t m = 0;
    for (uint32_t s = lo; s < hi; s++) m = h_len[s] > m ? h_len[s] : m;
    return m;
}

int glide_subgraph_build_and_merge(glide_ctx *ctx, const float *d_reorder_data, uint32_t reorder_num, uint32_t dim,
                                   const uint32_t *d_knn, uint32_t knn_degree, const uint32_t *h_segment_start,
                                   const uint32_t *h_segment_length, uint32_t S, const uint32_t *d_start_points_local,
                                   const uint32_t *d_map, uint32_t num, uint32_t graph_degree,
                                   const glide_search_params *p, float relaxant_factor, int metric, int skip_boundary,
                                   uint32_t *d_graph) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_reorder_data && d_knn && h_segment_start && h_segment_length && d_start_points_local && d_map && d_graph,
               GLIDE_ERR_BAD_ARG, "subgraph_build_and_merge: null pointer");
    GL_REQUIRE(ctx, S >= 1 && num <= reorder_num && dim > 0, GLIDE_ERR_BAD_ARG, "subgraph_build_and_merge: bad sizes");
    int rc = check_params(ctx, p, knn_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, graph_degree >= 1 && graph_degree <= 256, GLIDE_ERR_UNSUPPORTED, "Unsupported graph_degree");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    rc = ensure_ws(ctx, 2 * align256((size_t) S * 4));
    if (rc) return rc;
    Bump b(ctx->ws);
    uint32_t *d_start = b.take<uint32_t>(S), *d_len = b.take<uint32_t>(S);
    Timed timer(ctx);
    GL_CUDA(ctx, cudaMemcpyAsync(d_start, h_segment_start, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaMemcpyAsync(d_len, h_segment_length, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    BuildArgs a{};
    a.mode = kModeBuild;
    a.data = d_reorder_data; a.dim = dim; a.graph_in = d_knn; a.in_degree = knn_degree;
    a.graph_out = d_graph; a.out_degree = graph_degree;
    a.seg_start = d_start; a.seg_len = d_len; a.S = S; a.start_points = d_start_points_local; a.map = d_map;
    a.first = 0; a.count = num; a.alpha = relaxant_factor; a.metric = metric; a.p = to_host(p);
    a.counters = counters_or_null(ctx);
    a.max_seg_rows = longest_partition(h_segment_length, 0, S);
    GL_CUDA(ctx, launch_build(a, ctx->stream));
    const uint32_t boundary_num = reorder_num - num;
    if (!skip_boundary && boundary_num > 0) {  // glide_impl.cuh:149-187
        a.mode = kModeBoundary;
        a.fixed_segment = S - 1;
        a.max_seg_rows = h_segment_length[S - 1];
        a.first = num;
        a.count = boundary_num;
        GL_CUDA(ctx, launch_build(a, ctx->stream));
    }
    return timer.finish();
}

int glide_subgraph_build_range(glide_ctx *ctx, const float *d_reorder_data, uint32_t reorder_num, uint32_t dim,
                               const uint32_t *d_knn, uint32_t knn_degree, const uint32_t *h_segment_start,
                               const uint32_t *h_segment_length, uint32_t S, const uint32_t *d_start_points_local,
                               const uint32_t *d_map, uint32_t num, uint32_t graph_degree,
                               const glide_search_params *p, float relaxant_factor, int metric, uint32_t first_row,
                               uint32_t row_count, uint32_t *d_graph) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_reorder_data && d_knn && h_segment_start && h_segment_length && d_start_points_local && d_map && d_graph,
               GLIDE_ERR_BAD_ARG, "subgraph_build_range: null pointer");
    GL_REQUIRE(ctx, S >= 1 && num <= reorder_num && dim > 0, GLIDE_ERR_BAD_ARG, "subgraph_build_range: bad sizes");
    GL_REQUIRE(ctx, (uint64_t) first_row + row_count <= reorder_num, GLIDE_ERR_BAD_ARG, "subgraph_build_range: range beyond the rows");
    int rc = check_params(ctx, p, knn_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, graph_degree >= 1 && graph_degree <= 256, GLIDE_ERR_UNSUPPORTED, "Unsupported graph_degree");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    rc = ensure_ws(ctx, 2 * align256((size_t) S * 4));
    if (rc) return rc;
    Bump b(ctx->ws);
    uint32_t *d_start = b.take<uint32_t>(S), *d_len = b.take<uint32_t>(S);
    Timed timer(ctx);
    GL_CUDA(ctx, cudaMemcpyAsync(d_start, h_segment_start, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaMemcpyAsync(d_len, h_segment_length, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    BuildArgs a{};
    a.data = d_reorder_data; a.dim = dim; a.graph_in = d_knn; a.in_degree = knn_degree;
    a.graph_out = d_graph; a.out_degree = graph_degree;
    a.seg_start = d_start; a.seg_len = d_len; a.S = S; a.start_points = d_start_points_local; a.map = d_map;
    a.alpha = relaxant_factor; a.metric = metric; a.p = to_host(p);
    a.counters = counters_or_null(ctx);
    const uint32_t end = first_row + row_count;
    if (first_row < num) {  // main rows: build_kernel
        a.mode = kModeBuild;
        a.first = first_row;
        a.count = (end < num ? end : num) - first_row;
        a.max_seg_rows = longest_partition(h_segment_length, 0, S);
        GL_CUDA(ctx, launch_build(a, ctx->stream));
    }
    if (end > num) {  // boundary copies: build_boundary_kernel
        a.mode = kModeBoundary;
        a.fixed_segment = S - 1;
        a.first = first_row > num ? first_row : num;
        a.count = end - a.first;
        a.max_seg_rows = h_segment_length[S - 1];
        GL_CUDA(ctx, launch_build(a, ctx->stream));
    }
    return timer.finish();
}

int glide_subgraph_build_rows(glide_ctx *ctx, const float *d_reorder_data, uint32_t reorder_num, uint32_t dim,
                              const uint32_t *d_knn, uint32_t knn_degree, const uint32_t *h_segment_start,
                              const uint32_t *h_segment_length, uint32_t S, const uint32_t *d_start_points_local,
                              const uint32_t *d_map, uint32_t num, uint32_t graph_degree, const glide_search_params *p,
                              float relaxant_factor, int metric, uint32_t first_row, uint32_t row_count,
                              uint32_t *d_rows_out) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_reorder_data && d_knn && h_segment_start && h_segment_length && d_start_points_local && d_map && d_rows_out,
               GLIDE_ERR_BAD_ARG, "subgraph_build_rows: null pointer");
    GL_REQUIRE(ctx, S >= 1 && num <= reorder_num && dim > 0, GLIDE_ERR_BAD_ARG, "subgraph_build_rows: bad sizes");
    GL_REQUIRE(ctx, (uint64_t) first_row + row_count <= num, GLIDE_ERR_BAD_ARG,
               "subgraph_build_rows: the range must lie inside the non-boundary rows");
    int rc = check_params(ctx, p, knn_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, graph_degree >= 1 && graph_degree <= 256, GLIDE_ERR_UNSUPPORTED, "Unsupported graph_degree");
    if (row_count == 0) { ctx->last_ms = 0.0f; return GLIDE_OK; }
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    rc = ensure_ws(ctx, 2 * align256((size_t) S * 4));
    if (rc) return rc;
    Bump b(ctx->ws);
    uint32_t *d_start = b.take<uint32_t>(S), *d_len = b.take<uint32_t>(S);
    Timed timer(ctx);
    GL_CUDA(ctx, cudaMemcpyAsync(d_start, h_segment_start, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaMemcpyAsync(d_len, h_segment_length, (size_t) S * 4, cudaMemcpyHostToDevice, ctx->stream));
    BuildArgs a{};
    a.mode = kModeBuild;
    a.data = d_reorder_data; a.dim = dim; a.graph_in = d_knn; a.in_degree = knn_degree;
    a.graph_out = d_rows_out; a.out_first = first_row; a.rows_by_point = 1; a.out_degree = graph_degree;
    a.seg_start = d_start; a.seg_len = d_len; a.S = S; a.start_points = d_start_points_local; a.map = d_map;
    a.first = first_row; a.count = row_count;
    a.alpha = relaxant_factor; a.metric = metric; a.p = to_host(p);
    a.counters = counters_or_null(ctx);
    a.max_seg_rows = longest_partition(h_segment_length, 0, S);
    GL_CUDA(ctx, launch_build(a, ctx->stream));
    return timer.finish();
}

int glide_reverse_graph(glide_ctx *ctx, uint32_t *d_graph, uint32_t num, uint32_t graph_degree) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_graph && num > 0, GLIDE_ERR_BAD_ARG, "reverse_graph: bad argument");
    GL_REQUIRE(ctx, graph_degree >= 1 && graph_degree <= 256, GLIDE_ERR_UNSUPPORTED, "Unsupported graph_degree");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t need = 2 * align256((size_t) (num + 1) * 4) + align256((size_t) num * graph_degree * 8) +
                        align256(reverse_scan_tmp_bytes(num)) + 256;
    int rc = ensure_ws(ctx, need);
    if (rc) return rc;
    Bump b(ctx->ws);
    ReverseArgs a{};
    a.graph = d_graph; a.num = num; a.degree = graph_degree;
    a.counts = b.take<uint32_t>(num + 1);
    a.offsets = b.take<uint32_t>(num + 1);
    a.edges = b.take<unsigned long long>((size_t) num * graph_degree);
    a.scan_tmp = b.take<char>(reverse_scan_tmp_bytes(num));
    Timed timer(ctx);
    GL_CUDA(ctx, launch_reverse(a, ctx->stream));
    return timer.finish();
}

// Points of a refine launch in partition order: order[] lists 0..count-1 grouped by route[] (ascending
// index inside a group). The kernel results do not depend on the order in which points are
// processed (every point reads the snapshot and writes its own row); grouping makes the warps that
// run together walk the same part of the graph and of the data, which is what keeps the subgraph
// build in L2. Scratch: slot[count], totals[C+1], offsets[C+1], hist[slot_scratch_words], scan tmp.
struct OrderScratch {
    uint32_t *slot, *totals, *offsets, *hist, *order;
    void *scan_tmp;
};
size_t order_scratch_bytes(uint32_t count, uint32_t C) {
    return 2 * align256((size_t) count * 4) + 2 * align256((size_t) (C + 2) * 4) + align256(slot_scratch_words(count, C) * 4) +
           align256(scan_tmp_bytes(C + 1)) + 256;
}
OrderScratch carve_order_scratch(char *base, uint32_t count, uint32_t C) {
    OrderScratch o;
    o.slot = reinterpret_cast<uint32_t *>(base); base += align256((size_t) count * 4);
    o.order = reinterpret_cast<uint32_t *>(base); base += align256((size_t) count * 4);
    o.totals = reinterpret_cast<uint32_t *>(base); base += align256((size_t) (C + 2) * 4);
    o.offsets = reinterpret_cast<uint32_t *>(base); base += align256((size_t) (C + 2) * 4);
    o.hist = reinterpret_cast<uint32_t *>(base); base += align256(slot_scratch_words(count, C) * 4);
    o.scan_tmp = base;
    return o;
}
cudaError_t make_partition_order(const uint32_t *route, uint32_t count, uint32_t C, const OrderScratch &o, cudaStream_t st) {
    cudaError_t e = launch_slots(route, count, C, o.slot, o.totals, o.hist, st);
    if (e != cudaSuccess) return e;
    if ((e = exclusive_scan_u32(o.totals, C, o.offsets, o.scan_tmp, st)) != cudaSuccess) return e;
    return launch_scatter_members(route, o.slot, o.offsets, count, o.order, st);
}

// Points are refined in waves of wave_rows consecutive ids (0: one wave). Every search of a wave
// reads the graph as the waves before it left it; the wave's rows go to a staging buffer and are
// copied into the graph when the wave's kernel is done, so the result does not depend on the order
// in which warps run. The reference refines in place while other CTAs traverse the rows
// (graph_kernel.cuh:648, :660-671): a point there sees the rows of (roughly) all points with
// smaller ids already refined, which is what consecutive waves reproduce up to the wave size.
constexpr uint32_t kDefaultRefineWaveRows = 65536;

uint32_t default_refine_wave_rows() {
    static const uint32_t rows = [] {
        const char *e = std::getenv("GLIDE_B200_REFINE_WAVE");   // experiments: another wave size (0 = one wave)
        return e ? (uint32_t) std::strtoul(e, nullptr, 10) : kDefaultRefineWaveRows;
    }();
    return rows;
}

static int refine_common(glide_ctx *ctx, int mode, const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph,
                         uint32_t graph_degree, const float *d_centroids, uint32_t C, const uint32_t *d_start_points,
                         const glide_search_params *p, float relaxant_factor, int metric, uint32_t wave_rows) {
    GL_REQUIRE(ctx, d_data && d_graph && d_start_points && num > 0 && dim > 0, GLIDE_ERR_BAD_ARG, "refine: bad argument");
    int rc = check_params(ctx, p, graph_degree);
    if (rc) return rc;
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    if (wave_rows == 0 || wave_rows > num) wave_rows = num;
    const size_t stage_bytes = (size_t) wave_rows * graph_degree * 4;
    const bool routed = mode == kModeRefine;
    // work list of a wave: the rows with holes only (flags, list, count)
    const size_t list_bytes = 2 * align256((size_t) wave_rows * 4) + 256;
    rc = ensure_ws(ctx, align256(stage_bytes) + align256((size_t) num * 4) + list_bytes + (routed ? order_scratch_bytes(wave_rows, C) : 0));
    if (rc) return rc;
    uint32_t *staging = static_cast<uint32_t *>(ctx->ws);
    uint32_t *route = reinterpret_cast<uint32_t *>(static_cast<char *>(ctx->ws) + align256(stage_bytes));
    char *list_base = reinterpret_cast<char *>(route) + align256((size_t) num * 4);
    uint32_t *hole_flags = reinterpret_cast<uint32_t *>(list_base);
    uint32_t *hole_list = reinterpret_cast<uint32_t *>(list_base + align256((size_t) wave_rows * 4));
    uint32_t *hole_count = reinterpret_cast<uint32_t *>(list_base + 2 * align256((size_t) wave_rows * 4));
    Timed timer(ctx);
    OrderScratch o{};
    if (routed) {
        AssignArgs r{d_data, num, dim, d_centroids, C, -1.0f, metric, route, nullptr, C <= 4096 ? ctx->tc_norms : nullptr, nullptr};
        GL_CUDA(ctx, launch_assign(r, ctx->stream));
        o = carve_order_scratch(list_base + list_bytes, wave_rows, C);
    }
    unsigned long long *counters = counters_or_null(ctx);
    for (uint32_t lo = 0; lo < num; lo += wave_rows) {
        const uint32_t count = num - lo < wave_rows ? num - lo : wave_rows;
        BuildArgs a{};
        const uint32_t *grouped = nullptr;
        if (routed) {   // the wave's points grouped by partition: warps that run together share L2 lines
            GL_CUDA(ctx, make_partition_order(route + lo, count, C, o, ctx->stream));
            grouped = o.order;
        }
        // Rows without holes are copied as they are; the kernel gets the rows with holes only, as a
        // dense list, so that every warp of a CTA has a point to refine (with a warp per row of the
        // wave, a CTA keeps its registers until its one or two busy warps are done).
        GL_CUDA(ctx, cudaMemcpyAsync(staging, d_graph + (size_t) lo * graph_degree, (size_t) count * graph_degree * 4,
                                     cudaMemcpyDeviceToDevice, ctx->stream));
        GL_CUDA(ctx, launch_rows_with_holes(d_graph, lo, count, graph_degree, grouped, hole_flags, hole_list, hole_count, ctx->stream));
        a.order = hole_list;
        a.count_dev = hole_count;
        a.mode = mode;
        a.data = d_data; a.dim = dim; a.graph_in = d_graph; a.in_degree = graph_degree;
        a.graph_out = staging; a.out_first = lo; a.out_degree = graph_degree;
        a.start_points = d_start_points; a.centroids = d_centroids; a.C = C; a.route = route;
        a.first = lo; a.count = count; a.alpha = relaxant_factor; a.metric = metric; a.p = to_host(p);
        a.counters = counters;
        GL_CUDA(ctx, launch_build(a, ctx->stream));
        GL_CUDA(ctx, cudaMemcpyAsync(d_graph + (size_t) lo * graph_degree, staging, (size_t) count * graph_degree * 4,
                                     cudaMemcpyDeviceToDevice, ctx->stream));
    }
    return timer.finish();
}

int glide_refine_rows(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_graph,
                      uint32_t graph_degree, const float *d_centroids, uint32_t C, const uint32_t *d_start_points,
                      const glide_search_params *p, float relaxant_factor, int metric, uint32_t first, uint32_t count,
                      uint32_t *d_rows_out) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_data && d_graph && d_rows_out && d_centroids && d_start_points, GLIDE_ERR_BAD_ARG, "refine_rows: null pointer");
    GL_REQUIRE(ctx, num > 0 && dim > 0 && C >= 1 && (uint64_t) first + count <= num, GLIDE_ERR_BAD_ARG, "refine_rows: bad sizes");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroids_num");
    int rc = check_params(ctx, p, graph_degree);
    if (rc) return rc;
    if (count == 0) { ctx->last_ms = 0.0f; return GLIDE_OK; }
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t list_bytes = 2 * align256((size_t) count * 4) + 256;
    rc = ensure_ws(ctx, align256((size_t) count * 4) + list_bytes + order_scratch_bytes(count, C));
    if (rc) return rc;
    uint32_t *route = static_cast<uint32_t *>(ctx->ws);
    char *list_base = reinterpret_cast<char *>(route) + align256((size_t) count * 4);
    uint32_t *hole_flags = reinterpret_cast<uint32_t *>(list_base);
    uint32_t *hole_list = reinterpret_cast<uint32_t *>(list_base + align256((size_t) count * 4));
    uint32_t *hole_count = reinterpret_cast<uint32_t *>(list_base + 2 * align256((size_t) count * 4));
    Timed timer(ctx);
    AssignArgs r{d_data + (size_t) first * dim, count, dim, d_centroids, C, -1.0f, metric, route, nullptr, ctx->tc_norms, nullptr};
    GL_CUDA(ctx, launch_assign(r, ctx->stream));
    const OrderScratch o = carve_order_scratch(list_base + list_bytes, count, C);
    GL_CUDA(ctx, make_partition_order(route, count, C, o, ctx->stream));
    // as in refine_common: rows without holes are copied, the kernel works through the others as a dense list
    GL_CUDA(ctx, cudaMemcpyAsync(d_rows_out, d_graph + (size_t) first * graph_degree, (size_t) count * graph_degree * 4,
                                 cudaMemcpyDeviceToDevice, ctx->stream));
    GL_CUDA(ctx, launch_rows_with_holes(d_graph, first, count, graph_degree, o.order, hole_flags, hole_list, hole_count, ctx->stream));
    BuildArgs a{};
    a.order = hole_list;
    a.count_dev = hole_count;
    a.mode = kModeRefine;
    a.data = d_data; a.dim = dim; a.graph_in = d_graph; a.in_degree = graph_degree;
    a.graph_out = d_rows_out; a.out_first = first; a.out_degree = graph_degree;
    a.start_points = d_start_points; a.centroids = d_centroids; a.C = C; a.route = route; a.route_first = first;
    a.first = first; a.count = count; a.alpha = relaxant_factor; a.metric = metric; a.p = to_host(p);
    a.counters = counters_or_null(ctx);
    GL_CUDA(ctx, launch_build(a, ctx->stream));
    return timer.finish();
}

int glide_refine_waves(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph,
                       uint32_t graph_degree, const float *d_centroids, uint32_t C, const uint32_t *d_start_points,
                       const glide_search_params *p, float relaxant_factor, int metric, uint32_t wave_rows) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_centroids && C >= 1, GLIDE_ERR_BAD_ARG, "refine: centroids missing");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroids_num");
    return refine_common(ctx, kModeRefine, d_data, num, dim, d_graph, graph_degree, d_centroids, C, d_start_points, p,
                         relaxant_factor, metric, wave_rows);
}

int glide_refine(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph,
                 uint32_t graph_degree, const float *d_centroids, uint32_t C, const uint32_t *d_start_points,
                 const glide_search_params *p, float relaxant_factor, int metric) {
    return glide_refine_waves(ctx, d_data, num, dim, d_graph, graph_degree, d_centroids, C, d_start_points, p,
                              relaxant_factor, metric, default_refine_wave_rows());
}

// ---- search ----------------------------------------------------------------------------------
int glide_search(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_graph,
                 uint32_t graph_degree, const float *d_centroids, uint32_t C, const uint32_t *d_start_points,
                 const float *d_queries, uint32_t q, const glide_search_params *p, int metric, uint32_t *d_out_ids,
                 float *d_out_dists) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (q == 0) { ctx->last_ms = 0.0f; return GLIDE_OK; }  // an empty batch is valid and launches nothing
    GL_REQUIRE(ctx, d_data && d_graph && d_centroids && d_start_points && d_queries && d_out_ids && d_out_dists,
               GLIDE_ERR_BAD_ARG, "search: null pointer");
    GL_REQUIRE(ctx, num > 0 && dim > 0 && C >= 1, GLIDE_ERR_BAD_ARG, "search: zero size");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroids_num");
    int rc = check_params(ctx, p, graph_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, p->top_k >= 1 && p->top_k <= p->beam, GLIDE_ERR_BAD_ARG, "search: top_k must be in [1, beam]");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    // queries are handed out grouped by partition when the batch is large enough for that to matter
    const bool grouped = C > 1 && q >= 1024 && q <= 262144;
    rc = ensure_ws(ctx, 2 * align256((size_t) q * 4));
    if (rc) return rc;
    uint32_t *route = static_cast<uint32_t *>(ctx->ws);
    SearchArgs a{};
    a.data = d_data; a.graph = d_graph; a.degree = graph_degree; a.dim = dim;
    a.queries = d_queries; a.Q = q; a.top_k = p->top_k; a.metric = metric; a.p = to_host(p);
    a.centroids = d_centroids; a.C = C; a.start_points = d_start_points; a.route = route;
    a.out_ids = d_out_ids; a.out_dists = d_out_dists;
    a.counters = counters_or_null(ctx);
    a.ticket = ctx->ticket;
    Timed timer(ctx);
    AssignArgs r{d_queries, q, dim, d_centroids, C, -1.0f, metric, route, nullptr, ctx->tc_norms, a.counters ? a.counters + 3 : nullptr};
    uint32_t launched = 0;
    GL_CUDA(ctx, launch_assign(r, ctx->stream, &launched));
    if (grouped) {
        uint32_t *order = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(route) + align256((size_t) q * 4));
        GL_CUDA(ctx, launch_group_by_key(route, q, C, order, ctx->stream));
        a.order = order;
        launched += 1;
    }
    GL_CUDA(ctx, cudaEventRecord(ctx->ev_mid, ctx->stream));
    GL_CUDA(ctx, launch_search(a, ctx->stream));
    ctx->last_launches = launched + 1;
    rc = timer.finish();
    if (rc) return rc;
    cudaEventElapsedTime(&ctx->split_ms[0], ctx->ev_start, ctx->ev_mid);
    cudaEventElapsedTime(&ctx->split_ms[1], ctx->ev_mid, ctx->ev_stop);
    return GLIDE_OK;
}

int glide_search_host(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_graph,
                      uint32_t graph_degree, const float *d_centroids, uint32_t C, const uint32_t *d_start_points,
                      const float *h_queries, uint32_t q, const glide_search_params *p, int metric,
                      uint32_t *h_out_ids, float *h_out_dists) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (q == 0) { ctx->last_ms = 0.0f; return GLIDE_OK; }
    GL_REQUIRE(ctx, h_queries && h_out_ids && h_out_dists && p, GLIDE_ERR_BAD_ARG, "search_host: null pointer");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    // layout: [route and query order (used by glide_search)] [queries] [ids] [dists]
    const size_t route_b = 2 * align256((size_t) q * 4);
    const size_t qb = align256((size_t) q * dim * 4), rb = align256((size_t) q * p->top_k * 4);
    int rc = ensure_ws(ctx, route_b + qb + 2 * rb);
    if (rc) return rc;
    char *w = static_cast<char *>(ctx->ws) + route_b;
    float *d_q = reinterpret_cast<float *>(w);
    uint32_t *d_ids = reinterpret_cast<uint32_t *>(w + qb);
    float *d_dists = reinterpret_cast<float *>(w + qb + rb);
    // One batch, copies and kernels in stream order. Splitting the batch so that copies overlap the
    // kernels was measured slower: a search kernel over half the queries takes well over half the
    // time (per-query latency, not throughput, bounds a 5,000-query launch on this device).
    GL_CUDA(ctx, cudaMemcpyAsync(d_q, h_queries, (size_t) q * dim * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = glide_search(ctx, d_data, num, dim, d_graph, graph_degree, d_centroids, C, d_start_points, d_q, q, p, metric,
                      d_ids, d_dists);
    if (rc) return rc;
    GL_CUDA(ctx, cudaMemcpyAsync(h_out_ids, d_ids, (size_t) q * p->top_k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    GL_CUDA(ctx, cudaMemcpyAsync(h_out_dists, d_dists, (size_t) q * p->top_k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    GL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return GLIDE_OK;
}

// ---- host-buffer search, several batches in flight ---------------------------------------------
// glide_search_host blocks until its results are on the host, so the device idles while a batch
// crosses the host link in either direction. A pipe keeps `depth` batches in flight: uploads on
// one stream, the kernels of all batches in submission order on the context's stream, downloads
// on a third, tied together by events. Every batch has its own device buffers and routing scratch.
struct glide_search_pipe {
    glide_ctx *ctx = nullptr;
    uint32_t max_queries = 0, dim = 0, max_top_k = 0, depth = 0, next = 0;
    cudaStream_t up = nullptr, down = nullptr;
    struct Slot {
        float *d_q = nullptr;
        uint32_t *d_ids = nullptr, *d_route = nullptr;
        float *d_dists = nullptr;
        cudaEvent_t uploaded = nullptr, searched = nullptr, done = nullptr;
        bool busy = false;
    } slots[8];
};

int glide_search_pipe_create(glide_ctx *ctx, uint32_t max_queries, uint32_t dim, uint32_t max_top_k, uint32_t depth,
                             glide_search_pipe **out) {
    if (!ctx || !out) return GLIDE_ERR_BAD_ARG;
    *out = nullptr;
    GL_REQUIRE(ctx, max_queries >= 1 && dim >= 1 && max_top_k >= 1 && depth >= 1 && depth <= 8, GLIDE_ERR_BAD_ARG,
               "search_pipe_create: sizes must be positive and depth at most 8");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    auto *pipe = new glide_search_pipe;
    pipe->ctx = ctx; pipe->max_queries = max_queries; pipe->dim = dim; pipe->max_top_k = max_top_k; pipe->depth = depth;
    cudaError_t e = cudaStreamCreateWithFlags(&pipe->up, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&pipe->down, cudaStreamNonBlocking);
    for (uint32_t i = 0; i < depth && e == cudaSuccess; i++) {
        auto &sl = pipe->slots[i];
        e = cudaMalloc(&sl.d_q, (size_t) max_queries * dim * 4);
        if (e == cudaSuccess) e = cudaMalloc(&sl.d_ids, (size_t) max_queries * max_top_k * 4);
        if (e == cudaSuccess) e = cudaMalloc(&sl.d_dists, (size_t) max_queries * max_top_k * 4);
        if (e == cudaSuccess) e = cudaMalloc(&sl.d_route, 2 * align256((size_t) max_queries * 4));
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.uploaded, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.searched, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        glide_search_pipe_destroy(pipe);
        return fail(ctx, e == cudaErrorMemoryAllocation ? GLIDE_ERR_NO_MEMORY : GLIDE_ERR_CUDA, "search_pipe_create: %s",
                    cudaGetErrorString(e));
    }
    *out = pipe;
    return GLIDE_OK;
}

void glide_search_pipe_destroy(glide_search_pipe *pipe) {
    if (!pipe) return;
    cudaSetDevice(pipe->ctx->device);
    if (pipe->up) cudaStreamSynchronize(pipe->up);
    cudaStreamSynchronize(pipe->ctx->stream);
    if (pipe->down) cudaStreamSynchronize(pipe->down);
    for (auto &sl : pipe->slots) {
        cudaFree(sl.d_q); cudaFree(sl.d_ids); cudaFree(sl.d_dists); cudaFree(sl.d_route);
        if (sl.uploaded) cudaEventDestroy(sl.uploaded);
        if (sl.searched) cudaEventDestroy(sl.searched);
        if (sl.done) cudaEventDestroy(sl.done);
    }
    if (pipe->up) cudaStreamDestroy(pipe->up);
    if (pipe->down) cudaStreamDestroy(pipe->down);
    delete pipe;
}

int glide_search_pipe_wait(glide_search_pipe *pipe, uint32_t slot) {
    if (!pipe) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = pipe->ctx;
    GL_REQUIRE(ctx, slot < pipe->depth, GLIDE_ERR_BAD_ARG, "search_pipe_wait: no such slot");
    auto &sl = pipe->slots[slot];
    if (!sl.busy) return GLIDE_OK;
    sl.busy = false;
    GL_CUDA(ctx, cudaEventSynchronize(sl.done));
    return GLIDE_OK;
}

int glide_search_pipe_submit(glide_search_pipe *pipe, const float *d_data, uint32_t num, uint32_t dim,
                             const uint32_t *d_graph, uint32_t graph_degree, const float *d_centroids, uint32_t C,
                             const uint32_t *d_start_points, const float *h_queries, uint32_t q,
                             const glide_search_params *p, int metric, uint32_t *h_out_ids, float *h_out_dists,
                             uint32_t *slot_out) {
    if (!pipe) return GLIDE_ERR_BAD_ARG;
    glide_ctx *ctx = pipe->ctx;
    GL_REQUIRE(ctx, d_data && d_graph && d_centroids && d_start_points && h_queries && h_out_ids && h_out_dists && p && slot_out,
               GLIDE_ERR_BAD_ARG, "search_pipe_submit: null pointer");
    GL_REQUIRE(ctx, q >= 1 && q <= pipe->max_queries && dim == pipe->dim && num > 0 && C >= 1, GLIDE_ERR_BAD_ARG,
               "search_pipe_submit: batch larger than the pipe was made for, or another dim");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroids_num");
    int rc = check_params(ctx, p, graph_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, p->top_k >= 1 && p->top_k <= p->beam && p->top_k <= pipe->max_top_k, GLIDE_ERR_BAD_ARG,
               "search_pipe_submit: top_k must be in [1, beam] and within the pipe's max_top_k");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    const uint32_t slot = pipe->next;
    rc = glide_search_pipe_wait(pipe, slot);   // the slot's last batch has left its buffers
    if (rc) return rc;
    auto &sl = pipe->slots[slot];
    GL_CUDA(ctx, cudaMemcpyAsync(sl.d_q, h_queries, (size_t) q * dim * 4, cudaMemcpyHostToDevice, pipe->up));
    GL_CUDA(ctx, cudaEventRecord(sl.uploaded, pipe->up));
    GL_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, sl.uploaded, 0));
    SearchArgs a{};
    a.data = d_data; a.graph = d_graph; a.degree = graph_degree; a.dim = dim;
    a.queries = sl.d_q; a.Q = q; a.top_k = p->top_k; a.metric = metric; a.p = to_host(p);
    a.centroids = d_centroids; a.C = C; a.start_points = d_start_points; a.route = sl.d_route;
    a.out_ids = sl.d_ids; a.out_dists = sl.d_dists;
    a.ticket = ctx->ticket;
    AssignArgs r{sl.d_q, q, dim, d_centroids, C, -1.0f, metric, sl.d_route, nullptr, ctx->tc_norms, nullptr};
    uint32_t launched = 0;
    GL_CUDA(ctx, launch_assign(r, ctx->stream, &launched));
    if (C > 1 && q >= 1024 && q <= 262144) {
        uint32_t *order = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(sl.d_route) + align256((size_t) q * 4));
        GL_CUDA(ctx, launch_group_by_key(sl.d_route, q, C, order, ctx->stream));
        a.order = order;
        launched += 1;
    }
    GL_CUDA(ctx, launch_search(a, ctx->stream));
    ctx->last_launches = launched + 1;
    GL_CUDA(ctx, cudaEventRecord(sl.searched, ctx->stream));
    GL_CUDA(ctx, cudaStreamWaitEvent(pipe->down, sl.searched, 0));
    GL_CUDA(ctx, cudaMemcpyAsync(h_out_ids, sl.d_ids, (size_t) q * p->top_k * 4, cudaMemcpyDeviceToHost, pipe->down));
    GL_CUDA(ctx, cudaMemcpyAsync(h_out_dists, sl.d_dists, (size_t) q * p->top_k * 4, cudaMemcpyDeviceToHost, pipe->down));
    GL_CUDA(ctx, cudaEventRecord(sl.done, pipe->down));
    sl.busy = true;
    pipe->next = (slot + 1) % pipe->depth;
    *slot_out = slot;
    return GLIDE_OK;
}

// ---- search without any allocation -----------------------------------------------------------
// Some hosts must not allocate device memory at call time: a serving loop whose device memory
// is handed out once by its own pool and where a cudaMalloc would stall every stream of the
// device, or a process that runs close to the memory limit and cannot risk a growing scratch
// arena. glide_search needs one word of scratch per query (the partition each query is routed
// to); here that scratch is a fixed array inside the library image, so the call touches no
// allocator. Every GPU that loads the library carries the array until the process exits.
constexpr uint32_t kStaticRouteCapacity = 65536;  // queries per call (256 KB of device memory)
static __device__ __align__(256) uint32_t g_static_route[kStaticRouteCapacity];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<uint32_t *> g_static_route_ptr[kMaxDevices];  // device address of g_static_route, per device (zero-initialised)
}  // namespace

int glide_search_static_scratch(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim,
                                const uint32_t *d_graph, uint32_t graph_degree, const float *d_centroids, uint32_t C,
                                const uint32_t *d_start_points, const float *d_queries, uint32_t q,
                                const glide_search_params *p, int metric, uint32_t *d_out_ids, float *d_out_dists) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (q == 0) { ctx->last_ms = 0.0f; return GLIDE_OK; }
    GL_REQUIRE(ctx, q <= kStaticRouteCapacity, GLIDE_ERR_UNSUPPORTED,
               "search_static_scratch: more than 65536 queries in one call; split the batch or use glide_search");
    GL_REQUIRE(ctx, d_data && d_graph && d_centroids && d_start_points && d_queries && d_out_ids && d_out_dists,
               GLIDE_ERR_BAD_ARG, "search_static_scratch: null pointer");
    GL_REQUIRE(ctx, num > 0 && dim > 0 && C >= 1, GLIDE_ERR_BAD_ARG, "search_static_scratch: zero size");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroids_num");
    GL_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kMaxDevices, GLIDE_ERR_UNSUPPORTED,
               "search_static_scratch: device index beyond 63");
    int rc = check_params(ctx, p, graph_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, p->top_k >= 1 && p->top_k <= p->beam, GLIDE_ERR_BAD_ARG, "search: top_k must be in [1, beam]");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    // First call on this device: resolve the array's device address. In host code the symbol is
    // only a handle, never an address a kernel may use.
    uint32_t *route = g_static_route_ptr[ctx->device].load(std::memory_order_acquire);
    if (!route) {   // two threads may both resolve it: they store the same address
        void *addr = nullptr;
        GL_CUDA(ctx, cudaGetSymbolAddress(&addr, g_static_route));
        route = static_cast<uint32_t *>(addr);
        g_static_route_ptr[ctx->device].store(route, std::memory_order_release);
    }
    SearchArgs a{};
    a.data = d_data; a.graph = d_graph; a.degree = graph_degree; a.dim = dim;
    a.queries = d_queries; a.Q = q; a.top_k = p->top_k; a.metric = metric; a.p = to_host(p);
    a.centroids = d_centroids; a.C = C; a.start_points = d_start_points; a.route = route;
    a.out_ids = d_out_ids; a.out_dists = d_out_dists;
    a.counters = counters_or_null(ctx);
    Timed timer(ctx);
    // no scratch for the tensor-core prefilter here: this entry point keeps to the exact kernels
    AssignArgs r{d_queries, q, dim, d_centroids, C, -1.0f, metric, route, nullptr, nullptr, nullptr};
    uint32_t launched = 0;
    GL_CUDA(ctx, launch_assign(r, ctx->stream, &launched));
    GL_CUDA(ctx, cudaEventRecord(ctx->ev_mid, ctx->stream));
    GL_CUDA(ctx, launch_search(a, ctx->stream));
    ctx->last_launches = launched + 1;
    rc = timer.finish();
    if (rc) return rc;
    cudaEventElapsedTime(&ctx->split_ms[0], ctx->ev_start, ctx->ev_mid);
    cudaEventElapsedTime(&ctx->split_ms[1], ctx->ev_mid, ctx->ev_stop);
    return GLIDE_OK;
}

// ---- large path ------------------------------------------------------------------------------
int glide_select_segments(glide_ctx *ctx, const float *d_queries, uint32_t q, uint32_t dim, const float *d_centroids,
                          uint32_t C, uint32_t min_segment_num, float boundary_factor, int metric, uint32_t *d_out) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_queries && d_centroids && d_out && dim > 0 && C >= 1, GLIDE_ERR_BAD_ARG, "select_segments: bad argument");
    GL_REQUIRE(ctx, C <= 4096, GLIDE_ERR_UNSUPPORTED, "Unsupported centroid_size");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    SelectSegmentArgs a{d_queries, q, dim, d_centroids, C, min_segment_num, boundary_factor, metric, d_out};
    Timed timer(ctx);
    GL_CUDA(ctx, launch_select_segments(a, ctx->stream));
    return timer.finish();
}

int glide_search_on_sub(glide_ctx *ctx, const float *d_data, uint32_t dim, const uint32_t *d_graph,
                        uint32_t graph_degree, const uint32_t *d_map, uint32_t start_point, const float *d_queries,
                        uint32_t q, const uint32_t *d_segment_ids, uint32_t segment_num, uint32_t segment_id,
                        const glide_search_params *p, int metric, uint32_t *d_final_ids, float *d_final_dists) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_data && d_graph && d_map && d_queries && d_segment_ids && d_final_ids && d_final_dists,
               GLIDE_ERR_BAD_ARG, "search_on_sub: null pointer");
    int rc = check_params(ctx, p, graph_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, p->top_k >= 1 && p->top_k <= 128 && p->top_k <= p->beam, GLIDE_ERR_UNSUPPORTED, "Unsupported topk");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    SearchArgs a{};
    a.data = d_data; a.graph = d_graph; a.degree = graph_degree; a.dim = dim;
    a.queries = d_queries; a.Q = q; a.top_k = p->top_k; a.metric = metric; a.p = to_host(p);
    a.C = 1; a.out_ids = d_final_ids; a.out_dists = d_final_dists;
    a.segment_ids = d_segment_ids; a.segment_num = segment_num; a.segment_id = segment_id;
    a.start_point = start_point; a.map = d_map;
    a.counters = counters_or_null(ctx);
    a.ticket = ctx->ticket;
    Timed timer(ctx);
    GL_CUDA(ctx, launch_search(a, ctx->stream));
    return timer.finish();
}

int glide_build_partition(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, const uint32_t *d_knn,
                          uint32_t knn_degree, uint32_t start_point, uint32_t graph_degree,
                          const glide_search_params *p, float relaxant_factor, int metric, uint32_t *d_graph) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_REQUIRE(ctx, d_data && d_knn && d_graph && num > 0 && dim > 0, GLIDE_ERR_BAD_ARG, "build_partition: bad argument");
    int rc = check_params(ctx, p, knn_degree);
    if (rc) return rc;
    GL_REQUIRE(ctx, graph_degree >= 1 && graph_degree <= 256, GLIDE_ERR_UNSUPPORTED, "Unsupported graph_degree");
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    rc = ensure_ws(ctx, 3 * 256);
    if (rc) return rc;
    Bump b(ctx->ws);
    uint32_t *d_start = b.take<uint32_t>(1), *d_len = b.take<uint32_t>(1), *d_sp = b.take<uint32_t>(1);
    const uint32_t zero = 0;
    Timed timer(ctx);
    GL_CUDA(ctx, cudaMemcpyAsync(d_start, &zero, 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaMemcpyAsync(d_len, &num, 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaMemcpyAsync(d_sp, &start_point, 4, cudaMemcpyHostToDevice, ctx->stream));
    BuildArgs a{};
    a.mode = kModeBuild;
    a.data = d_data; a.dim = dim; a.graph_in = d_knn; a.in_degree = knn_degree;
    a.graph_out = d_graph; a.out_degree = graph_degree;
    a.seg_start = d_start; a.seg_len = d_len; a.S = 1; a.start_points = d_sp; a.map = nullptr;
    a.first = 0; a.count = num; a.alpha = relaxant_factor; a.metric = metric; a.p = to_host(p);
    a.counters = counters_or_null(ctx);
    a.max_seg_rows = num;
    GL_CUDA(ctx, launch_build(a, ctx->stream));
    return timer.finish();
}

int glide_refine_partition(glide_ctx *ctx, const float *d_data, uint32_t num, uint32_t dim, uint32_t *d_graph,
                           uint32_t graph_degree, uint32_t start_point, const glide_search_params *p,
                           float relaxant_factor, int metric) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    GL_CUDA(ctx, cudaSetDevice(ctx->device));
    // the start point travels in the context's own device word (ordered before the kernels on the stream)
    GL_CUDA(ctx, cudaMemcpyAsync(ctx->start_point_word, &start_point, 4, cudaMemcpyHostToDevice, ctx->stream));
    GL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // `start_point` is a stack variable of this call
    return refine_common(ctx, kModeRefineRow, d_data, num, dim, d_graph, graph_degree, nullptr, 1, ctx->start_point_word,
                         p, relaxant_factor, metric, default_refine_wave_rows());
}

}  // extern "C"
