// C++ host mirror of the reference's LARGE path, header-only over the C ABI (glide_b200.h):
// preprocess_for_large (partition.cuh:417-447), build_knn_for_large (nn_descent.cuh:1515-1581)
// and GLIDE_large (glide_large.cuh:14-212, glide_large_impl.cuh:14-507). The data set lives in
// host memory; one partition at a time is resident on the GPU.
//
// What a caller of the reference will notice: rows are fp32 (the reference's large path is
// uint8), every random choice takes a seed, no trailing rows are dropped (the reference
// processes floor(N / batch_num) * batch_num rows, partition.cuh:231), and partitions keep the
// rows in ascending original id.
#pragma once

#include <limits>
#include <numeric>

#include "glide_b200.hpp"

namespace glide_b200 {

namespace detail {
// rows grouped by partition, ascending row id inside a partition
inline void group_by_partition(const HostMatrix<float> &h_data, const uint32_t *nearest, uint32_t C,
                               HostMatrix<float> &h_reorder_data, std::vector<uint32_t> &h_map,
                               std::vector<uint32_t> &h_segment_start, std::vector<uint32_t> &h_segment_length) {
    const uint32_t n = h_data.rows, dim = h_data.cols;
    h_segment_length.assign(C, 0);
    for (uint32_t i = 0; i < n; i++) h_segment_length[nearest[i]]++;
    h_segment_start.assign(C, 0);
    for (uint32_t c = 1; c < C; c++) h_segment_start[c] = h_segment_start[c - 1] + h_segment_length[c - 1];
    std::vector<uint32_t> cursor(h_segment_start);
    h_map.assign(n, 0);
    h_reorder_data = HostMatrix<float>(n, dim);
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t pos = cursor[nearest[i]]++;
        h_map[pos] = i;
        std::copy_n(h_data.data_handle() + (size_t) i * dim, dim, h_reorder_data.data_handle() + (size_t) pos * dim);
    }
}
}  // namespace detail

// Centroids from a host-gathered sample (farthest-first + Lloyd on the GPU), nearest-centroid
// assignment batch by batch (no boundary test, partition_kernel.cuh:122-162), then the rows
// grouped by partition. h_segment_start / h_segment_length get centroid_num entries.
inline void preprocess_for_large(const Context &ctx, const PartitionParameter &param, const HostMatrix<float> &h_data,
                                 HostMatrix<float> &h_reorder_data, std::vector<uint32_t> &h_map,
                                 std::vector<uint32_t> &h_segment_start, std::vector<uint32_t> &h_segment_length,
                                 HostMatrix<float> &h_centroids, uint32_t batch_num, const std::string &result_file,
                                 uint64_t seed = 0) {
    const uint32_t n = h_data.rows, dim = h_data.cols, C = param.centroid_num;
    if (n == 0 || dim == 0 || C == 0) throw std::invalid_argument("preprocess_for_large: empty input");
    float seconds = 0.0f;
    // sample -> k-means
    const uint32_t sample_num = std::max<uint32_t>(C, (uint32_t) ((double) n * param.sample_factor));
    std::vector<uint32_t> ids(sample_num);
    if (glide_sample_ids(n, sample_num, seed, ids.data()) != GLIDE_OK) throw std::invalid_argument("sample_ids: bad argument");
    HostMatrix<float> sample(sample_num, dim);
    for (uint32_t i = 0; i < sample_num; i++)
        std::copy_n(h_data.data_handle() + (size_t) ids[i] * dim, dim, sample.data_handle() + (size_t) i * dim);
    DeviceBuffer<float> d_sample(ctx, sample.data_handle(), sample.size());
    DeviceBuffer<float> d_centroids(ctx, (size_t) C * dim);
    uint32_t rounds = 0;
    ctx.check(glide_kmeans_fit(ctx.get(), d_sample.data_handle(), sample_num, dim, C, 0, (int) param.metric, 1,
                               d_centroids.data_handle(), nullptr, &rounds));
    seconds += ctx.last_kernel_seconds();
    d_sample.reset();
    // assignment, batch by batch
    const uint32_t batch = (n + std::max(1u, batch_num) - 1) / std::max(1u, batch_num);
    std::vector<uint32_t> nearest(n);
    DeviceBuffer<float> d_rows(ctx, (size_t) batch * dim);
    DeviceBuffer<uint32_t> d_index(ctx, (size_t) batch * 3);
    std::vector<uint32_t> index((size_t) batch * 3), tmp_start(C + 1), tmp_len(C + 1);
    for (uint32_t lo = 0; lo < n; lo += batch) {
        const uint32_t cnt = std::min(batch, n - lo);
        d_rows.upload(h_data.data_handle() + (size_t) lo * dim, (size_t) cnt * dim);
        ctx.check(glide_define_partition(ctx.get(), d_rows.data_handle(), cnt, dim, d_centroids.data_handle(), C, -1.0f,
                                         (int) param.metric, d_index.data_handle(), tmp_start.data(), tmp_len.data()));
        seconds += ctx.last_kernel_seconds();
        d_index.download(index.data(), (size_t) cnt * 3);
        for (uint32_t i = 0; i < cnt; i++) nearest[lo + i] = index[(size_t) i * 3];
    }
    detail::group_by_partition(h_data, nearest.data(), C, h_reorder_data, h_map, h_segment_start, h_segment_length);
    h_centroids = HostMatrix<float>(C, dim);
    d_centroids.download(h_centroids.data_handle(), h_centroids.size());
    std::printf("preprocessing time: %g s\n", seconds);
    if (!result_file.empty()) append_result(result_file, stream_text(seconds) + ",");
}

// The same from a matrix file (the reference's main loads the file first, large_preprocess.cu:56,
// row by row, load.cuh:23-26): the sample rows are read with a few seeks, k-means gives the
// centroids, then glide_load_rows streams the file into pinned memory with several reader threads
// while the GPU assigns the chunks already read. Same outputs as loading the file and calling
// preprocess_for_large; h_data receives the rows in file order.
inline void preprocess_for_large(const Context &ctx, const PartitionParameter &param, const std::string &data_file,
                                 HostMatrix<float> &h_data, HostMatrix<float> &h_reorder_data, std::vector<uint32_t> &h_map,
                                 std::vector<uint32_t> &h_segment_start, std::vector<uint32_t> &h_segment_length,
                                 HostMatrix<float> &h_centroids, const std::string &result_file, uint64_t seed = 0) {
    uint32_t n = 0, dim = 0;
    if (glide_matrix_file_info(data_file.c_str(), 4, &n, &dim) != GLIDE_OK) throw std::runtime_error("Cannot read file " + data_file);
    const uint32_t C = param.centroid_num;
    if (n == 0 || dim == 0 || C == 0) throw std::invalid_argument("preprocess_for_large: empty input");
    float seconds = 0.0f;
    const uint32_t sample_num = std::max<uint32_t>(C, (uint32_t) ((double) n * param.sample_factor));
    std::vector<uint32_t> ids(sample_num);
    if (glide_sample_ids(n, sample_num, seed, ids.data()) != GLIDE_OK) throw std::invalid_argument("sample_ids: bad argument");
    HostMatrix<float> sample(sample_num, dim);
    {
        std::ifstream in(data_file, std::ios::binary);
        for (uint32_t i = 0; i < sample_num; i++) {
            in.seekg((std::streamoff) (8 + (uint64_t) ids[i] * dim * 4));
            in.read(reinterpret_cast<char *>(sample.data_handle() + (size_t) i * dim), (std::streamsize) dim * 4);
        }
        if (!in) throw std::runtime_error(data_file + ": truncated");
    }
    DeviceBuffer<float> d_sample(ctx, sample.data_handle(), sample.size());
    DeviceBuffer<float> d_centroids(ctx, (size_t) C * dim);
    uint32_t rounds = 0;
    ctx.check(glide_kmeans_fit(ctx.get(), d_sample.data_handle(), sample_num, dim, C, 0, (int) param.metric, 1,
                               d_centroids.data_handle(), nullptr, &rounds));
    seconds += ctx.last_kernel_seconds();
    d_sample.reset();
    h_data = HostMatrix<float>(n, dim);
    std::vector<uint32_t> nearest(n);
    const bool pinned = glide_host_register(h_data.data_handle(), h_data.size() * sizeof(float)) == GLIDE_OK;
    double stats[3] = {0, 0, 0};
    const int rc = glide_load_rows(ctx.get(), data_file.c_str(), 4, 0, n, h_data.data_handle(), 0, 0, d_centroids.data_handle(), C,
                                   (int) param.metric, nearest.data(), stats);
    if (pinned) glide_host_unregister(h_data.data_handle());
    ctx.check(rc);
    detail::group_by_partition(h_data, nearest.data(), C, h_reorder_data, h_map, h_segment_start, h_segment_length);
    h_centroids = HostMatrix<float>(C, dim);
    d_centroids.download(h_centroids.data_handle(), h_centroids.size());
    std::printf("preprocessing time: %g s (file read and assignment, overlapped: %g s)\n", seconds, stats[1]);
    if (!result_file.empty()) append_result(result_file, stream_text(seconds) + ",");
}

// kNN graph of every partition, one resident partition at a time; partition-local ids.
inline HostMatrix<int> build_knn_for_large(const Context &ctx, const NNDescentParameter &param,
                                           const HostMatrix<float> &h_reorder_data,
                                           const std::vector<uint32_t> &h_segment_start,
                                           const std::vector<uint32_t> &h_segment_length, const std::string &result_file,
                                           Metric metric = Metric::Euclidean, uint64_t seed = 0) {
    const uint32_t dim = h_reorder_data.cols;
    const uint32_t degree = std::min(param.graph_degree, param.intermediate_graph_degree);
    HostMatrix<int> knn(h_reorder_data.rows, degree);
    float seconds = 0.0f;
    for (size_t s = 0; s < h_segment_start.size(); s++) {
        const uint32_t start = h_segment_start[s], len = h_segment_length[s];
        if (len == 0) continue;
        DeviceBuffer<float> d_part(ctx, h_reorder_data.data_handle() + (size_t) start * dim, (size_t) len * dim);
        DeviceBuffer<int> d_knn(ctx, (size_t) len * degree);
        const uint32_t zero = 0;
        uint32_t rounds = 0;
        ctx.check(glide_build_nnd(ctx.get(), d_part.data_handle(), len, dim, &zero, &len, 1, degree, param.max_iterations,
                                  param.termination_threshold, 0, 0xffffffffu, seed, (int) metric, d_knn.data_handle(), &rounds));
        seconds += ctx.last_kernel_seconds();
        d_knn.download(knn.data_handle() + (size_t) start * degree, (size_t) len * degree);
    }
    std::printf("knn time: %g s\n", seconds);
    if (!result_file.empty()) append_result(result_file, stream_text(seconds) + ",");
    return knn;
}

// Host-resident index over disjoint partitions.
class GLIDE_large {
public:
    GLIDE_large(const Context &ctx, uint32_t graph_degree, Metric metric, HostMatrix<float> h_reorder_data,
                std::vector<uint32_t> h_map, HostMatrix<float> h_centroids, std::vector<uint32_t> h_segment_start,
                std::vector<uint32_t> h_segment_length)
        : ctx_(ctx), metric_(metric), degree_(graph_degree), data_(std::move(h_reorder_data)), map_(std::move(h_map)),
          centroids_(std::move(h_centroids)), seg_start_(std::move(h_segment_start)), seg_len_(std::move(h_segment_length)),
          graph_(data_.rows, graph_degree), start_points_(seg_start_.size(), 0) {
        std::fill(graph_.v.begin(), graph_.v.end(), 0xffffffffu);
    }
    uint32_t num() const { return data_.rows; }
    uint32_t dim() const { return data_.cols; }
    uint32_t graph_degree() const { return degree_; }
    uint32_t segment_num() const { return (uint32_t) seg_start_.size(); }
    uint32_t centroids_num() const { return centroids_.rows; }
    const HostMatrix<uint32_t> &graph_view() const { return graph_; }
    const std::vector<uint32_t> &start_point_view() const { return start_points_; }

    void load(const HostMatrix<uint32_t> &h_graph, const std::vector<uint32_t> &h_start_points) {
        if (h_graph.rows != data_.rows || h_graph.cols != degree_) throw std::invalid_argument("graph shape does not match the index");
        if (h_start_points.size() != seg_start_.size()) throw std::invalid_argument("one start point per partition expected");
        std::copy(h_graph.v.begin(), h_graph.v.end(), graph_.v.begin());   // in place: the buffer may be page-locked
        start_points_ = h_start_points;
    }

    // one seeded member per partition, as a partition-local id (glide_large_impl.cuh:50-77)
    void start_point_select(uint64_t seed) {
        uint64_t state = seed;
        for (size_t i = 0; i < seg_len_.size(); i++) {
            state += 0x9E3779B97F4A7C15ull;
            uint64_t z = state;
            z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
            z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
            z ^= z >> 31;
            start_points_[i] = seg_len_[i] ? (uint32_t) (z % seg_len_[i]) : 0u;
        }
    }

    // GLIDE_large::build (glide_large_impl.cuh:79-328) through the library's streaming object: rows
    // and kNN rows of partition p + 1 are uploaded while partition p runs build_for_large_kernel,
    // reverse edges and refine_for_large_kernel, and the rows of partition p - 1 are downloaded.
    void build(const IndexParameter &build_param, const SearchParameter &search_param_knn,
               const SearchParameter &search_param_refine, const HostMatrix<int> &h_knn_graph, const std::string &result_file,
               uint64_t seed = 0) {
        if (h_knn_graph.rows != data_.rows) throw std::invalid_argument("kNN graph rows do not match the data");
        const glide_search_params pk = search_param_knn.c(), pr = search_param_refine.c();
        std::vector<uint32_t> parts(seg_start_.size());
        for (size_t i = 0; i < parts.size(); i++) parts[i] = (uint32_t) i;
        glide_large *h = handle();
        ctx_.check(glide_large_build(h, parts.data(), (uint32_t) parts.size(), h_knn_graph.cols, &pk, &pr, build_param.relaxant_factor,
                                     0, -1.0f, 0, 0xffffffffu, seed, h_knn_graph.data_handle(), nullptr));
        ctx_.check(glide_large_get_start_points(h, start_points_.data()));
        double st[8];
        glide_large_last_stats(h, st);
        const double seconds = st[1] + st[2] + st[3];
        std::printf("index build time: %g s\n", seconds);
        if (!result_file.empty()) append_result(result_file, stream_text(seconds) + ",");
    }

    // glide_large_impl.cuh:355-507: route every query to the partitions within boundary_factor of
    // its nearest centroid (at least min_segment_num), search each partition some query is routed to,
    // fold into a running top-k. Result ids are original row ids. resident_budget_bytes > 0 keeps
    // partitions in device memory across calls.
    void search(const SearchParameter &param, uint32_t min_segment_num, float boundary_factor, const HostMatrix<float> &h_query,
                HostMatrix<uint32_t> &result_ids, HostMatrix<float> &result_dists, const std::string &result_file,
                size_t resident_budget_bytes = 0) {
        const glide_search_params p = param.c();
        const uint32_t q = h_query.rows;
        std::vector<uint32_t> parts(seg_start_.size());
        for (size_t i = 0; i < parts.size(); i++) parts[i] = (uint32_t) i;
        glide_large *h = handle();
        ctx_.check(glide_large_set_start_points(h, start_points_.data()));
        if (resident_budget_bytes) ctx_.check(glide_large_make_resident(h, parts.data(), (uint32_t) parts.size(), resident_budget_bytes, nullptr));
        DeviceBuffer<float> d_query(ctx_, h_query.data_handle(), h_query.size());
        DeviceBuffer<float> d_centroids(ctx_, centroids_.data_handle(), centroids_.size());
        DeviceBuffer<uint32_t> d_ids(ctx_, (size_t) q * param.top_k);
        DeviceBuffer<float> d_dists(ctx_, (size_t) q * param.top_k);
        ctx_.check(glide_large_search(h, d_query.data_handle(), q, d_centroids.data_handle(), centroids_.rows, min_segment_num,
                                      boundary_factor, &p, parts.data(), (uint32_t) parts.size(), d_ids.data_handle(),
                                      d_dists.data_handle()));
        double st[8];
        glide_large_last_stats(h, st);
        const double seconds = st[0] + st[1];
        std::printf("query time: %g s   QPS: %g\n", seconds, q / seconds);
        if (!result_file.empty()) append_result(result_file, stream_text(seconds) + "," + stream_text(q / seconds) + ",");
        result_ids = HostMatrix<uint32_t>(q, param.top_k);
        result_dists = HostMatrix<float>(q, param.top_k);
        d_ids.download(result_ids.data_handle(), result_ids.size());
        d_dists.download(result_dists.data_handle(), result_dists.size());
    }

    // build_with_merge is declared in the reference (glide_large.cuh:96) and defined nowhere; here:
    // the ordinary build without refine, every partition kept in device memory, then
    // glide_large_merge (links across partition borders within boundary_factor, reverse edges over
    // the whole graph). search_merged then runs one beam search per query on the merged graph.
    void build_with_merge(const IndexParameter &build_param, const SearchParameter &search_param_knn,
                          const HostMatrix<int> &h_knn_graph, const std::string &result_file, float boundary_factor = 1.2f,
                          uint32_t link_count = 8, uint64_t seed = 0) {
        SearchParameter no_refine;
        no_refine.beam = 0;
        build(build_param, search_param_knn, no_refine, h_knn_graph, "", seed);
        std::vector<uint32_t> parts(seg_start_.size());
        for (size_t i = 0; i < parts.size(); i++) parts[i] = (uint32_t) i;
        glide_large *h = handle();
        uint32_t kept = 0;
        ctx_.check(glide_large_make_resident(h, parts.data(), (uint32_t) parts.size(), ~(size_t) 0, &kept));
        SearchParameter link;
        link.top_k = link_count;
        link.beam = 32;
        derive_search_params(link, degree_);
        const glide_search_params pl = link.c();
        DeviceBuffer<float> d_centroids(ctx_, centroids_.data_handle(), centroids_.size());
        double st[3] = {0, 0, 0};
        ctx_.check(glide_large_merge(h, d_centroids.data_handle(), centroids_.rows, boundary_factor, link_count, &pl, st));
        std::printf("merge time: %g s (%u rows with links)\n", st[0] + st[1], (unsigned) st[2]);
        if (!result_file.empty()) append_result(result_file, stream_text(st[0] + st[1]) + ",");
    }

    void search_merged(const SearchParameter &param, const HostMatrix<float> &h_query, HostMatrix<uint32_t> &result_ids,
                       HostMatrix<float> &result_dists) {
        const glide_search_params p = param.c();
        const uint32_t q = h_query.rows;
        DeviceBuffer<float> d_query(ctx_, h_query.data_handle(), h_query.size());
        DeviceBuffer<float> d_centroids(ctx_, centroids_.data_handle(), centroids_.size());
        DeviceBuffer<uint32_t> d_ids(ctx_, (size_t) q * param.top_k);
        DeviceBuffer<float> d_dists(ctx_, (size_t) q * param.top_k);
        ctx_.check(glide_large_search_merged(handle(), d_query.data_handle(), q, d_centroids.data_handle(), centroids_.rows, &p,
                                             d_ids.data_handle(), d_dists.data_handle()));
        result_ids = HostMatrix<uint32_t>(q, param.top_k);
        result_dists = HostMatrix<float>(q, param.top_k);
        d_ids.download(result_ids.data_handle(), result_ids.size());
        d_dists.download(result_dists.data_handle(), result_dists.size());
    }

    ~GLIDE_large() {
        if (large_) {
            glide_large_destroy(large_);
            glide_host_unregister(data_.data_handle());
            glide_host_unregister(graph_.data_handle());
        }
    }
    GLIDE_large(const GLIDE_large &) = delete;
    GLIDE_large &operator=(const GLIDE_large &) = delete;

private:
    const Context &ctx_;
    Metric metric_;
    uint32_t degree_;
    HostMatrix<float> data_;
    std::vector<uint32_t> map_;
    HostMatrix<float> centroids_;
    std::vector<uint32_t> seg_start_, seg_len_;
    HostMatrix<uint32_t> graph_;
    std::vector<uint32_t> start_points_;
    glide_large *large_ = nullptr;

    // the streaming object over this index's host buffers, made on first use (the buffers are
    // page-locked in place so that uploads and downloads run asynchronously)
    glide_large *handle() {
        if (!large_) {
            glide_host_register(data_.data_handle(), data_.size() * sizeof(float));
            glide_host_register(graph_.data_handle(), graph_.size() * sizeof(uint32_t));
            ctx_.check(glide_large_create(ctx_.get(), data_.data_handle(), 0, data_.cols, seg_start_.data(), seg_len_.data(),
                                          (uint32_t) seg_start_.size(), map_.data(), degree_, (int) metric_, graph_.data_handle(),
                                          &large_));
        }
        return large_;
    }
};

}  // namespace glide_b200
