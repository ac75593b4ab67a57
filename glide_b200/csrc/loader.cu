// Matrix files into pinned host memory, overlapped with partition assignment.
//
// The reference reads a matrix file one row at a time through an ifstream into pageable memory
// (load.cuh:10-30) and only then starts to work on it. Here a few reader threads pull the file in
// with large positional reads straight into the caller's (pinned) destination, and every chunk is
// uploaded and assigned to its nearest centroid (what define_partition_for_large_kernel,
// partition_kernel.cuh:122-162, computes per batch) while the chunks after it are still being
// read: file, host link and GPU work at the same time. uint8 files cross the host link as bytes
// and are widened on the device.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>
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

double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// reads exactly `bytes` at `offset`; false on error or a short file
bool read_fully(int fd, char *dst, size_t bytes, uint64_t offset) {
    while (bytes > 0) {
        const ssize_t got = pread(fd, dst, std::min<size_t>(bytes, (size_t) 1 << 30), (off_t) offset);
        if (got < 0 && errno == EINTR) continue;
        if (got <= 0) return false;
        dst += got;
        offset += (uint64_t) got;
        bytes -= (size_t) got;
    }
    return true;
}

struct Chunks {
    std::mutex m;
    std::condition_variable cv;
    std::vector<char> done;   // 0 pending, 1 read, 2 failed
    std::atomic<uint32_t> next{0};
};

struct DeviceSide {
    cudaStream_t up = nullptr;
    cudaEvent_t uploaded[2] = {nullptr, nullptr}, assigned[2] = {nullptr, nullptr};
    void *raw[2] = {nullptr, nullptr};      // chunk as it is in the file
    float *rows[2] = {nullptr, nullptr};    // fp32 rows (== raw for fp32 files)
    uint32_t *nearest = nullptr;
    ~DeviceSide() {
        for (int s = 0; s < 2; s++) {
            if (rows[s] && rows[s] != raw[s]) cudaFree(rows[s]);
            if (raw[s]) cudaFree(raw[s]);
            if (uploaded[s]) cudaEventDestroy(uploaded[s]);
            if (assigned[s]) cudaEventDestroy(assigned[s]);
        }
        if (nearest) cudaFree(nearest);
        if (up) cudaStreamDestroy(up);
    }
};

}  // namespace

extern "C" {

int glide_matrix_file_info(const char *path, uint32_t elem_bytes, uint32_t *rows, uint32_t *dim) {
    if (!path || !rows || !dim || (elem_bytes != 1 && elem_bytes != 4)) return GLIDE_ERR_BAD_ARG;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return GLIDE_ERR_IO;
    uint32_t head[2] = {0, 0};
    struct stat st;
    const bool ok = read_fully(fd, reinterpret_cast<char *>(head), 8, 0) && fstat(fd, &st) == 0;
    close(fd);
    if (!ok) return GLIDE_ERR_IO;
    // load.cuh:16-19: u32 rows, u32 dim, then the rows
    if ((uint64_t) st.st_size < 8 + (uint64_t) head[0] * head[1] * elem_bytes) return GLIDE_ERR_IO;
    *rows = head[0];
    *dim = head[1];
    return GLIDE_OK;
}

int glide_load_rows(glide_ctx *ctx, const char *path, uint32_t elem_bytes, uint64_t first_row, uint64_t rows, void *h_rows,
                    uint32_t chunk_rows, uint32_t threads, const float *d_centroids, uint32_t centroid_num, int metric,
                    uint32_t *h_nearest, double *stats) {
    if (!ctx) return GLIDE_ERR_BAD_ARG;
    if (!path || !h_rows || (elem_bytes != 1 && elem_bytes != 4))
        return fail(ctx, GLIDE_ERR_BAD_ARG, "load_rows: null pointer or element size other than 1 and 4");
    if ((d_centroids != nullptr) != (h_nearest != nullptr) || (d_centroids && centroid_num == 0))
        return fail(ctx, GLIDE_ERR_BAD_ARG, "load_rows: centroids and the output for partition ids go together");
    uint32_t file_rows = 0, dim = 0;
    int rc = glide_matrix_file_info(path, elem_bytes, &file_rows, &dim);
    if (rc) return fail(ctx, rc, "load_rows: cannot read %s (missing, or shorter than its header says)", path);
    if (first_row + rows > file_rows || dim == 0) return fail(ctx, GLIDE_ERR_BAD_ARG, "load_rows: rows beyond the end of the file");
    if (d_centroids && elem_bytes == 1 && dim % 4 != 0)
        return fail(ctx, GLIDE_ERR_UNSUPPORTED, "load_rows: uint8 rows need dim %% 4 == 0 for the assignment");
    if (stats) stats[0] = stats[1] = stats[2] = 0.0;
    if (rows == 0) return GLIDE_OK;
    if (chunk_rows == 0) chunk_rows = (uint32_t) std::max<uint64_t>(1, ((uint64_t) 64 << 20) / ((uint64_t) dim * elem_bytes));
    if (threads == 0) threads = 4;
    threads = std::min<uint32_t>(threads, 64);
    const uint64_t row_bytes = (uint64_t) dim * elem_bytes;
    const uint32_t K = (uint32_t) ((rows + chunk_rows - 1) / chunk_rows);
    if ((uint64_t) K * chunk_rows >> 40) return fail(ctx, GLIDE_ERR_BAD_ARG, "load_rows: too many rows");

    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(ctx, GLIDE_ERR_IO, "load_rows: cannot open %s", path);
    posix_fadvise(fd, 0, 0, POSIX_FADV_SEQUENTIAL);

    Chunks ch;
    ch.done.assign(K, 0);
    std::atomic<double> read_end{0.0};
    const double t0 = now_s();
    auto reader = [&]() {
        for (;;) {
            const uint32_t k = ch.next.fetch_add(1);
            if (k >= K) return;
            const uint64_t lo = (uint64_t) k * chunk_rows, cnt = std::min<uint64_t>(chunk_rows, rows - lo);
            const bool ok = read_fully(fd, static_cast<char *>(h_rows) + lo * row_bytes, cnt * row_bytes,
                                       8 + (first_row + lo) * row_bytes);
            {
                std::lock_guard<std::mutex> g(ch.m);
                ch.done[k] = ok ? 1 : 2;
            }
            ch.cv.notify_all();
            double seen = read_end.load();
            const double t = now_s();
            while (t > seen && !read_end.compare_exchange_weak(seen, t)) {}
        }
    };
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < std::min(threads, K); t++) pool.emplace_back(reader);
    auto join_all = [&]() {
        for (auto &t : pool) t.join();
        close(fd);
    };
    auto wait_chunk = [&](uint32_t k) {
        std::unique_lock<std::mutex> g(ch.m);
        ch.cv.wait(g, [&] { return ch.done[k] != 0; });
        return ch.done[k] == 1;
    };

    double waited = 0.0;
    cudaError_t e = cudaSuccess;
    bool io_ok = true;
    if (!d_centroids) {
        for (uint32_t k = 0; k < K && io_ok; k++) io_ok = wait_chunk(k);
    } else {
        DeviceSide dv;
        e = cudaSetDevice(ctx->device);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&dv.up, cudaStreamNonBlocking);
        for (int s = 0; s < 2 && e == cudaSuccess; s++) {
            e = cudaMalloc(&dv.raw[s], (size_t) chunk_rows * row_bytes);
            if (e == cudaSuccess && elem_bytes == 1) e = cudaMalloc(&dv.rows[s], (size_t) chunk_rows * dim * 4);
            if (elem_bytes == 4) dv.rows[s] = static_cast<float *>(dv.raw[s]);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&dv.uploaded[s], cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&dv.assigned[s], cudaEventDisableTiming);
        }
        if (e == cudaSuccess) e = cudaMalloc(&dv.nearest, (size_t) rows * 4);
        for (uint32_t k = 0; k < K && e == cudaSuccess && io_ok; k++) {
            const int s = (int) (k & 1u);
            const uint64_t lo = (uint64_t) k * chunk_rows, cnt = std::min<uint64_t>(chunk_rows, rows - lo);
            const double w0 = now_s();
            io_ok = wait_chunk(k);
            waited += now_s() - w0;
            if (!io_ok) break;
            if (k >= 2) e = cudaStreamWaitEvent(dv.up, dv.assigned[s], 0);   // the slot's last chunk has been consumed
            if (e == cudaSuccess)
                e = cudaMemcpyAsync(dv.raw[s], static_cast<char *>(h_rows) + lo * row_bytes, cnt * row_bytes,
                                    cudaMemcpyHostToDevice, dv.up);
            if (e == cudaSuccess) e = cudaEventRecord(dv.uploaded[s], dv.up);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, dv.uploaded[s], 0);
            if (e == cudaSuccess && elem_bytes == 1)
                e = glide::launch_widen_u8(static_cast<const uint8_t *>(dv.raw[s]), dv.rows[s], (size_t) cnt * dim, ctx->stream);
            if (e == cudaSuccess) {
                glide::AssignArgs a{dv.rows[s], (uint32_t) cnt, dim, d_centroids, centroid_num, -1.0f, metric,
                                    dv.nearest + lo, nullptr, ctx->tc_norms, nullptr};
                e = glide::launch_assign(a, ctx->stream);
            }
            if (e == cudaSuccess) e = cudaEventRecord(dv.assigned[s], ctx->stream);
        }
        if (e == cudaSuccess && io_ok)
            e = cudaMemcpyAsync(h_nearest, dv.nearest, (size_t) rows * 4, cudaMemcpyDeviceToHost, ctx->stream);
        const cudaError_t e2 = cudaStreamSynchronize(ctx->stream);   // before the buffers go away, whatever happened
        if (dv.up) cudaStreamSynchronize(dv.up);
        if (e == cudaSuccess) e = e2;
    }
    // a failed chunk leaves the other readers running to the end of their chunks; wait for them
    join_all();
    const double t1 = now_s();
    if (stats) {
        stats[0] = read_end.load() - t0;   // until the last chunk was in host memory
        stats[1] = t1 - t0;                // until the partition ids were in host memory
        stats[2] = waited;                 // time the device side spent waiting for the file
    }
    if (!io_ok) return fail(ctx, GLIDE_ERR_IO, "load_rows: read error in %s", path);
    if (e != cudaSuccess)
        return fail(ctx, e == cudaErrorMemoryAllocation ? GLIDE_ERR_NO_MEMORY : GLIDE_ERR_CUDA, "load_rows: %s", cudaGetErrorString(e));
    return GLIDE_OK;
}

}  // extern "C"
