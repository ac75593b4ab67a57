// C++ host mirror of the reference's API for the small path, header-only over the C ABI
// (glide_b200.h). Names, argument meaning and error behaviour follow the reference:
// params.cuh (Metric, PartitionParameter, NNDescentParameter, IndexParameter, SearchParameter,
// calculate_hash_bitlen, calculate_hash_reset_interval, adjust_search_params), load.cuh (file
// formats), partition.cuh:159-193 (preprocess), nn_descent.cuh:1405-1467 (build_nnd),
// glide.cuh:14-189 (GLIDE). RAFT views are replaced by the small HostMatrix / DeviceBuffer types
// below; everything that was seeded from std::random_device takes a seed.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <stdexcept>
#include <sstream>
#include <string>
#include <vector>

#include "glide_b200.h"

namespace glide_b200 {

enum class Metric { Euclidean = GLIDE_METRIC_EUCLIDEAN, Cosine = GLIDE_METRIC_COSINE };  // params.cuh:5-8

inline Metric parse_metric(const std::string &name) {  // small_build.cu:55-59
    if (name == "Euclidean") return Metric::Euclidean;
    if (name == "Cosine") return Metric::Cosine;
    throw std::invalid_argument("unknown metric '" + name + "' (expected Euclidean or Cosine)");
}

struct PartitionParameter {  // params.cuh:10-15
    uint32_t centroid_num = 10;
    float boundary_factor = 1.05f;
    float sample_factor = 0.01f;
    Metric metric = Metric::Euclidean;
};

struct NNDescentParameter {  // params.cuh:17-25
    uint32_t graph_degree = 64;
    uint32_t intermediate_graph_degree = 128;
    uint32_t max_iterations = 20;
    float termination_threshold = 0.0001f;
    explicit NNDescentParameter(size_t degree)
        : graph_degree((uint32_t) degree), intermediate_graph_degree((uint32_t) (1.5 * degree)) {}
};

struct IndexParameter {  // params.cuh:27-35
    uint32_t graph_degree = 32;
    uint32_t knn_degree = 32;
    float relaxant_factor = 1.05f;
    Metric metric = Metric::Euclidean;
};

struct SearchParameter {  // params.cuh:37-47
    uint32_t top_k = 10;
    uint32_t beam = 100;
    uint32_t max_iterations = 0;
    uint32_t min_iterations = 0;
    uint32_t hash_bit = 0;
    float hash_max_fill_rate = 0.5f;
    uint32_t hashmap_min_bitlen = 0;
    uint32_t hash_reset_interval = 1;
    uint32_t search_block_size = 0;
    glide_search_params c() const { return {top_k, beam, max_iterations, min_iterations, hash_bit, hash_reset_interval}; }
};

inline uint32_t calculate_hash_bitlen(uint32_t beam, uint32_t graph_degree, float fill, uint32_t min_bitlen) {
    return glide_calculate_hash_bitlen(beam, graph_degree, fill, min_bitlen);
}
inline uint32_t calculate_hash_reset_interval(uint32_t beam, uint32_t graph_degree, float fill, uint32_t bitlen) {
    return glide_calculate_hash_reset_interval(beam, graph_degree, fill, bitlen);
}
inline void adjust_search_params(uint32_t min_iterations, uint32_t &max_iterations, uint32_t &beam) {
    glide_adjust_search_params(min_iterations, &max_iterations, &beam);
}
// what every reference main does after filling beam (small_build.cu:61-82, small_search.cu:98-107)
inline void derive_search_params(SearchParameter &p, uint32_t degree_for_hash) {
    adjust_search_params(p.min_iterations, p.max_iterations, p.beam);
    p.hash_bit = calculate_hash_bitlen(p.beam, degree_for_hash, p.hash_max_fill_rate, p.hashmap_min_bitlen);
    p.hash_reset_interval = calculate_hash_reset_interval(p.beam, degree_for_hash, p.hash_max_fill_rate, p.hash_bit);
}

// ---- host containers and files (load.cuh) ------------------------------------------------
template<typename T>
struct HostMatrix {
    uint32_t rows = 0, cols = 0;
    std::vector<T> v;
    HostMatrix() = default;
    HostMatrix(uint32_t r, uint32_t c) : rows(r), cols(c), v((size_t) r * c) {}
    T *data_handle() { return v.data(); }
    const T *data_handle() const { return v.data(); }
    uint32_t extent(int i) const { return i == 0 ? rows : cols; }
    size_t size() const { return v.size(); }
    T &operator()(uint32_t i, uint32_t j) { return v[(size_t) i * cols + j]; }
    const T &operator()(uint32_t i, uint32_t j) const { return v[(size_t) i * cols + j]; }
};

// The reference prints a message and carries on when a file cannot be opened (load.cuh:12-14);
// here that and a short file throw.
template<typename T>
HostMatrix<T> load_matrix_data(const std::string &file) {  // load.cuh:10-30
    std::ifstream in(file, std::ios::binary);
    if (!in) throw std::runtime_error("Cannot open file " + file);
    uint32_t n = 0, dim = 0;
    in.read(reinterpret_cast<char *>(&n), 4);
    in.read(reinterpret_cast<char *>(&dim), 4);
    if (!in) throw std::runtime_error(file + ": missing 8-byte header");
    HostMatrix<T> m(n, dim);
    in.read(reinterpret_cast<char *>(m.v.data()), (std::streamsize) (m.v.size() * sizeof(T)));
    if ((size_t) in.gcount() != m.v.size() * sizeof(T)) throw std::runtime_error(file + ": truncated");
    return m;
}
template<typename T>
void save_matrix_data(const std::string &file, const HostMatrix<T> &m) {  // load.cuh:90-103
    std::ofstream out(file, std::ios::binary);
    if (!out) throw std::runtime_error("Cannot open file " + file);
    out.write(reinterpret_cast<const char *>(&m.rows), 4);
    out.write(reinterpret_cast<const char *>(&m.cols), 4);
    out.write(reinterpret_cast<const char *>(m.v.data()), (std::streamsize) (m.v.size() * sizeof(T)));
}
inline void load_segment(const std::string &file, std::vector<uint32_t> &start, std::vector<uint32_t> &length) {
    std::ifstream in(file, std::ios::binary);  // load.cuh:33-68
    if (!in) throw std::runtime_error("Cannot open file " + file);
    uint32_t s = 0;
    in.read(reinterpret_cast<char *>(&s), 4);
    start.resize(s);
    length.resize(s);
    in.read(reinterpret_cast<char *>(start.data()), (std::streamsize) s * 4);
    in.read(reinterpret_cast<char *>(length.data()), (std::streamsize) s * 4);
    if (!in) throw std::runtime_error(file + ": truncated");
}
inline void save_segment(const std::string &file, const std::vector<uint32_t> &start, const std::vector<uint32_t> &length) {
    std::ofstream out(file, std::ios::binary);  // load.cuh:106-117
    if (!out) throw std::runtime_error("Cannot open file " + file);
    const uint32_t s = (uint32_t) start.size();
    out.write(reinterpret_cast<const char *>(&s), 4);
    out.write(reinterpret_cast<const char *>(start.data()), (std::streamsize) s * 4);
    out.write(reinterpret_cast<const char *>(length.data()), (std::streamsize) s * 4);
}
inline std::vector<uint32_t> load_vector_data(const std::string &file) {  // load.cuh:71-86
    std::ifstream in(file, std::ios::binary);
    if (!in) throw std::runtime_error("Cannot open file " + file);
    uint32_t n = 0;
    in.read(reinterpret_cast<char *>(&n), 4);
    std::vector<uint32_t> v(n);
    in.read(reinterpret_cast<char *>(v.data()), (std::streamsize) n * 4);
    if (!in) throw std::runtime_error(file + ": truncated");
    return v;
}
inline void save_vector_data(const std::string &file, const std::vector<uint32_t> &v) {  // load.cuh:120-127
    std::ofstream out(file, std::ios::binary);
    if (!out) throw std::runtime_error("Cannot open file " + file);
    const uint32_t n = (uint32_t) v.size();
    out.write(reinterpret_cast<const char *>(&n), 4);
    out.write(reinterpret_cast<const char *>(v.data()), (std::streamsize) n * 4);
}

// ---- context and device memory -------------------------------------------------------------
class Context {
public:
    explicit Context(int device = 0) {
        if (glide_ctx_create(device, &ctx_) != GLIDE_OK) throw std::runtime_error("glide_ctx_create failed (no usable GPU?)");
    }
    ~Context() { glide_ctx_destroy(ctx_); }
    Context(const Context &) = delete;
    Context &operator=(const Context &) = delete;
    glide_ctx *get() const { return ctx_; }
    // CUDA failures throw like RAFT_CUDA_TRY; unsupported shapes throw std::invalid_argument
    // (kernel_config.cuh:47-48, :59-60)
    void check(int rc) const {
        if (rc == GLIDE_OK) return;
        if (rc == GLIDE_ERR_UNSUPPORTED) throw std::invalid_argument(glide_last_error(ctx_));
        throw std::runtime_error(glide_last_error(ctx_));
    }
    float last_kernel_seconds() const { return glide_last_kernel_ms(ctx_) / 1000.0f; }

private:
    glide_ctx *ctx_ = nullptr;
};

template<typename T>
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    DeviceBuffer(const Context &ctx, size_t count) : ctx_(&ctx), count_(count) {
        void *p = nullptr;
        ctx.check(glide_malloc(ctx.get(), count * sizeof(T), &p));
        ptr_ = static_cast<T *>(p);
    }
    DeviceBuffer(const Context &ctx, const T *host, size_t count) : DeviceBuffer(ctx, count) { upload(host, count); }
    ~DeviceBuffer() { reset(); }
    DeviceBuffer(DeviceBuffer &&o) noexcept : ctx_(o.ctx_), ptr_(o.ptr_), count_(o.count_) { o.ptr_ = nullptr; o.count_ = 0; }
    DeviceBuffer &operator=(DeviceBuffer &&o) noexcept {
        if (this != &o) { reset(); ctx_ = o.ctx_; ptr_ = o.ptr_; count_ = o.count_; o.ptr_ = nullptr; o.count_ = 0; }
        return *this;
    }
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    void reset() { if (ptr_) glide_free(ptr_); ptr_ = nullptr; count_ = 0; }   // the reference frees consumed inputs
    void adopt(const Context &ctx, T *p, size_t count) { reset(); ctx_ = &ctx; ptr_ = p; count_ = count; }
    void upload(const T *host, size_t count) { ctx_->check(glide_memcpy_h2d(ctx_->get(), ptr_, host, count * sizeof(T))); }
    void download(T *host, size_t count) const { ctx_->check(glide_memcpy_d2h(ctx_->get(), host, ptr_, count * sizeof(T))); }
    void fill_u32(uint32_t value) { ctx_->check(glide_memset_u32(ctx_->get(), reinterpret_cast<uint32_t *>(ptr_), value, count_ * sizeof(T) / 4)); }
    T *data_handle() const { return ptr_; }
    size_t size() const { return count_; }

private:
    const Context *ctx_ = nullptr;
    T *ptr_ = nullptr;
    size_t count_ = 0;
};

// Numbers go into result files the way the reference streams them (`file << value`, e.g.
// small_search.cu:121-126): "0.9514", not std::to_string's "0.951400".
template<typename T>
inline std::string stream_text(T value) {
    std::ostringstream out;
    out << value;
    return out.str();
}

inline void append_result(const std::string &file, const std::string &text) {
    std::ofstream out(file, std::ios::app);
    out << text;
}

// ---- preprocess (partition.cuh:159-193) ----------------------------------------------------
// d_reorder_data and d_map are emplaced like the reference's std::optional outputs;
// h_segment_start / h_segment_length get centroid_num + 1 entries. Appends "<seconds>," to
// result_file as the reference does (:189-192).
inline void preprocess(const Context &ctx, const PartitionParameter &param, const DeviceBuffer<float> &d_data,
                       uint32_t num, uint32_t dim, DeviceBuffer<float> &d_reorder_data, DeviceBuffer<uint32_t> &d_map,
                       std::vector<uint32_t> &h_segment_start, std::vector<uint32_t> &h_segment_length,
                       DeviceBuffer<float> &d_centroids, uint32_t &reorder_num, const std::string &result_file,
                       uint64_t seed = 0) {
    h_segment_start.assign(param.centroid_num + 1, 0);
    h_segment_length.assign(param.centroid_num + 1, 0);
    d_centroids = DeviceBuffer<float>(ctx, (size_t) param.centroid_num * dim);
    float *reorder = nullptr;
    uint32_t *map = nullptr;
    ctx.check(glide_preprocess(ctx.get(), d_data.data_handle(), num, dim, param.centroid_num, param.boundary_factor,
                               param.sample_factor, (int) param.metric, seed, d_centroids.data_handle(),
                               h_segment_start.data(), h_segment_length.data(), &reorder, &map, &reorder_num));
    d_reorder_data.adopt(ctx, reorder, (size_t) reorder_num * dim);
    d_map.adopt(ctx, map, reorder_num);
    const float seconds = ctx.last_kernel_seconds();
    std::printf("preprocessing time: %g s\n", seconds);
    if (!result_file.empty()) append_result(result_file, stream_text(seconds) + ",");
}

// ---- build_nnd (nn_descent.cuh:1405-1467) ---------------------------------------------------
// Consumes d_data like the reference (data.reset(), :1257) when `consume` is set. Returns the
// rows x graph_degree int matrix of partition-local ids.
inline HostMatrix<int> build_nnd(const Context &ctx, const NNDescentParameter &param, DeviceBuffer<float> &d_data,
                                 uint32_t num, uint32_t dim, const std::vector<uint32_t> &h_segment_start,
                                 const std::vector<uint32_t> &h_segment_length, const std::string &result_file,
                                 Metric metric = Metric::Euclidean, uint64_t seed = 0, bool consume = false) {
    const uint32_t degree = std::min(param.graph_degree, param.intermediate_graph_degree);  // :1423-1425
    DeviceBuffer<int> d_knn(ctx, (size_t) num * degree);
    uint32_t rounds = 0;
    ctx.check(glide_build_nnd(ctx.get(), d_data.data_handle(), num, dim, h_segment_start.data(), h_segment_length.data(),
                              (uint32_t) h_segment_start.size(), degree, param.max_iterations,
                              param.termination_threshold, 0, 0xffffffffu, seed, (int) metric, d_knn.data_handle(), &rounds));
    const float seconds = ctx.last_kernel_seconds();
    if (consume) d_data.reset();
    HostMatrix<int> out(num, degree);
    d_knn.download(out.data_handle(), out.size());
    std::printf("knn time: %g s\n", seconds);
    if (!result_file.empty()) append_result(result_file, stream_text(seconds) + ",");
    return out;
}

// ---- GLIDE (glide.cuh:14-189, glide_impl.cuh:15-454) ---------------------------------------
class GLIDE {
public:
    // ctor uploads data and centroids (glide_impl.cuh:15-29)
    GLIDE(const Context &ctx, uint32_t graph_degree, const HostMatrix<float> &h_data, const HostMatrix<float> &h_centroids,
          Metric metric)
        : ctx_(ctx), metric_(metric), num_(h_data.rows), dim_(h_data.cols), degree_(graph_degree),
          centroid_num_(h_centroids.rows), d_data_(ctx, h_data.data_handle(), h_data.size()),
          d_centroids_(ctx, h_centroids.data_handle(), h_centroids.size()), d_graph_(ctx, (size_t) h_data.rows * graph_degree) {
        d_graph_.fill_u32(0xffffffffu);
    }
    uint32_t num() const { return num_; }
    uint32_t dim() const { return dim_; }
    uint32_t graph_degree() const { return degree_; }
    uint32_t centroid_num() const { return centroid_num_; }
    uint32_t start_point_num() const { return (uint32_t) d_start_points_.size(); }
    const DeviceBuffer<uint32_t> &graph_view() const { return d_graph_; }
    const DeviceBuffer<uint32_t> &start_point_view() const { return d_start_points_; }

    void load(const HostMatrix<uint32_t> &h_graph, const std::vector<uint32_t> &h_start_points) {  // :31-41
        if (h_graph.rows != num_ || h_graph.cols != degree_) throw std::invalid_argument("graph shape does not match the index");
        d_graph_.upload(h_graph.data_handle(), h_graph.size());
        d_start_points_ = DeviceBuffer<uint32_t>(ctx_, h_start_points.data(), h_start_points.size());
    }

    // GLIDE::build (glide_impl.cuh:319-368). The device inputs are consumed (reset) as there.
    void build(const IndexParameter &build_param, SearchParameter &search_param_knn, SearchParameter &search_param_refine,
               DeviceBuffer<int> &d_knn_graph, const std::vector<uint32_t> &h_segment_start,
               const std::vector<uint32_t> &h_segment_length, DeviceBuffer<uint32_t> &d_map,
               const std::vector<uint32_t> &h_map, DeviceBuffer<float> &d_reorder_data, uint32_t reorder_num,
               const std::string &result_file, uint64_t seed = 0) {
        const uint32_t S = (uint32_t) h_segment_start.size();
        std::vector<uint32_t> local(S), original(S > 1 ? S - 1 : 1);
        if (glide_start_point_select(h_segment_start.data(), h_segment_length.data(), S, h_map.data(), seed, local.data(),
                                     original.data()) != GLIDE_OK)
            throw std::invalid_argument("start_point_select: bad argument");
        DeviceBuffer<uint32_t> d_local(ctx_, local.data(), S);
        float build_time = 0.0f;
        const glide_search_params pk = search_param_knn.c();
        d_graph_.fill_u32(0xffffffffu);
        ctx_.check(glide_subgraph_build_and_merge(ctx_.get(), d_reorder_data.data_handle(), reorder_num, dim_,
                                                  reinterpret_cast<const uint32_t *>(d_knn_graph.data_handle()),
                                                  build_param.knn_degree, h_segment_start.data(), h_segment_length.data(), S,
                                                  d_local.data_handle(), d_map.data_handle(), num_, degree_, &pk,
                                                  build_param.relaxant_factor, (int) metric_, 0, d_graph_.data_handle()));
        build_time += ctx_.last_kernel_seconds();
        d_knn_graph.reset(); d_map.reset(); d_reorder_data.reset();           // :347-351
        original.resize(S - 1);
        d_start_points_ = DeviceBuffer<uint32_t>(ctx_, original.data(), original.size());  // :353-356
        ctx_.check(glide_reverse_graph(ctx_.get(), d_graph_.data_handle(), num_, degree_));
        build_time += ctx_.last_kernel_seconds();
        if (search_param_refine.beam != 0) {                                   // :360-362
            const glide_search_params pr = search_param_refine.c();
            ctx_.check(glide_refine(ctx_.get(), d_data_.data_handle(), num_, dim_, d_graph_.data_handle(), degree_,
                                    d_centroids_.data_handle(), centroid_num_, d_start_points_.data_handle(), &pr,
                                    build_param.relaxant_factor, (int) metric_));
            build_time += ctx_.last_kernel_seconds();
        }
        std::printf("index build time: %g s\n", build_time);
        if (!result_file.empty()) append_result(result_file, stream_text(build_time) + ",");
    }

    // GLIDE::search (glide_impl.cuh:370-454): host queries in, host results out
    void search(const SearchParameter &param, const HostMatrix<float> &h_query, HostMatrix<uint32_t> &result_ids,
                HostMatrix<float> &result_dists, const std::string &result_file) {
        const glide_search_params p = param.c();
        DeviceBuffer<float> d_query(ctx_, h_query.data_handle(), h_query.size());
        DeviceBuffer<uint32_t> d_ids(ctx_, (size_t) h_query.rows * param.top_k);
        DeviceBuffer<float> d_dists(ctx_, (size_t) h_query.rows * param.top_k);
        ctx_.check(glide_search(ctx_.get(), d_data_.data_handle(), num_, dim_, d_graph_.data_handle(), degree_,
                                d_centroids_.data_handle(), centroid_num_, d_start_points_.data_handle(),
                                d_query.data_handle(), h_query.rows, &p, (int) metric_, d_ids.data_handle(),
                                d_dists.data_handle()));
        const float seconds = ctx_.last_kernel_seconds();
        std::printf("query time: %g s   QPS: %g\n", seconds, h_query.rows / seconds);
        if (!result_file.empty()) append_result(result_file, stream_text(seconds) + "," + stream_text(h_query.rows / seconds) + ",");
        result_ids = HostMatrix<uint32_t>(h_query.rows, param.top_k);
        result_dists = HostMatrix<float>(h_query.rows, param.top_k);
        d_ids.download(result_ids.data_handle(), result_ids.size());
        d_dists.download(result_dists.data_handle(), result_dists.size());
    }

private:
    const Context &ctx_;
    Metric metric_;
    uint32_t num_, dim_, degree_, centroid_num_;
    DeviceBuffer<float> d_data_, d_centroids_;
    DeviceBuffer<uint32_t> d_graph_, d_start_points_;
};

// small_search.cu:14-36
inline float calculate_recall(const HostMatrix<uint32_t> &neighbors, const HostMatrix<uint32_t> &truth, uint32_t top_k) {
    float total = 0.0f;
    for (uint32_t q = 0; q < neighbors.rows; q++) {
        uint32_t correct = 0;
        for (uint32_t k = 0; k < top_k; k++)
            for (uint32_t t = 0; t < top_k; t++)
                if (truth(q, t) == neighbors(q, k)) { correct++; break; }
        total += (float) correct / top_k;
    }
    std::printf("total_recall: %g\n", total / neighbors.rows);
    return total / neighbors.rows;
}

}  // namespace glide_b200
