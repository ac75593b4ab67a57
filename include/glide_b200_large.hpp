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
    // group by partition, ascending row id inside a partition
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
    h_centroids = HostMatrix<float>(C, dim);
    d_centroids.download(h_centroids.data_handle(), h_centroids.size());
    std::printf("preprocessing time: %g s\n", seconds);
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
        graph_ = h_graph;
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

    // per resident partition: rows and kNN rows in, build_for_large_kernel, reverse edges,
    // refine_for_large_kernel, graph rows out (glide_large_impl.cuh:79-328)
    void build(const IndexParameter &build_param, const SearchParameter &search_param_knn,
               const SearchParameter &search_param_refine, const HostMatrix<int> &h_knn_graph, const std::string &result_file,
               uint64_t seed = 0) {
        if (h_knn_graph.rows != data_.rows) throw std::invalid_argument("kNN graph rows do not match the data");
        start_point_select(seed);
        const glide_search_params pk = search_param_knn.c(), pr = search_param_refine.c();
        const uint32_t dim = data_.cols, kd = h_knn_graph.cols;
        float seconds = 0.0f;
        for (size_t s = 0; s < seg_start_.size(); s++) {
            const uint32_t start = seg_start_[s], len = seg_len_[s];
            if (len == 0) continue;
            DeviceBuffer<float> d_part(ctx_, data_.data_handle() + (size_t) start * dim, (size_t) len * dim);
            DeviceBuffer<uint32_t> d_knn(ctx_, reinterpret_cast<const uint32_t *>(h_knn_graph.data_handle()) + (size_t) start * kd,
                                         (size_t) len * kd);
            DeviceBuffer<uint32_t> d_graph(ctx_, (size_t) len * degree_);
            d_graph.fill_u32(0xffffffffu);
            ctx_.check(glide_build_partition(ctx_.get(), d_part.data_handle(), len, dim, d_knn.data_handle(), kd, start_points_[s],
                                             degree_, &pk, build_param.relaxant_factor, (int) metric_, d_graph.data_handle()));
            seconds += ctx_.last_kernel_seconds();
            ctx_.check(glide_reverse_graph(ctx_.get(), d_graph.data_handle(), len, degree_));
            seconds += ctx_.last_kernel_seconds();
            if (search_param_refine.beam != 0) {
                ctx_.check(glide_refine_partition(ctx_.get(), d_part.data_handle(), len, dim, d_graph.data_handle(), degree_,
                                                  start_points_[s], &pr, build_param.relaxant_factor, (int) metric_));
                seconds += ctx_.last_kernel_seconds();
            }
            d_graph.download(graph_.data_handle() + (size_t) start * degree_, (size_t) len * degree_);
        }
        std::printf("index build time: %g s\n", seconds);
        if (!result_file.empty()) append_result(result_file, stream_text(seconds) + ",");
    }

    // glide_large_impl.cuh:355-507: route every query to the partitions within boundary_factor of
    // its nearest centroid (at least min_segment_num), search each resident partition, fold into a
    // running top-k. Result ids are original row ids.
    void search(const SearchParameter &param, uint32_t min_segment_num, float boundary_factor, const HostMatrix<float> &h_query,
                HostMatrix<uint32_t> &result_ids, HostMatrix<float> &result_dists, const std::string &result_file) {
        const glide_search_params p = param.c();
        const uint32_t q = h_query.rows, dim = data_.cols, S = segment_num();
        DeviceBuffer<float> d_query(ctx_, h_query.data_handle(), h_query.size());
        DeviceBuffer<float> d_centroids(ctx_, centroids_.data_handle(), centroids_.size());
        DeviceBuffer<uint32_t> d_routes(ctx_, (size_t) q * centroids_.rows);
        ctx_.check(glide_select_segments(ctx_.get(), d_query.data_handle(), q, dim, d_centroids.data_handle(), centroids_.rows,
                                         min_segment_num, boundary_factor, (int) metric_, d_routes.data_handle()));
        float seconds = ctx_.last_kernel_seconds();
        DeviceBuffer<uint32_t> d_ids(ctx_, (size_t) q * param.top_k);
        d_ids.fill_u32(0xffffffffu);
        std::vector<float> init((size_t) q * param.top_k, std::numeric_limits<float>::max());
        DeviceBuffer<float> d_dists(ctx_, init.data(), init.size());
        for (uint32_t s = 0; s < S; s++) {
            const uint32_t start = seg_start_[s], len = seg_len_[s];
            if (len == 0) continue;
            DeviceBuffer<float> d_part(ctx_, data_.data_handle() + (size_t) start * dim, (size_t) len * dim);
            DeviceBuffer<uint32_t> d_graph(ctx_, graph_.data_handle() + (size_t) start * degree_, (size_t) len * degree_);
            DeviceBuffer<uint32_t> d_map(ctx_, map_.data() + start, len);
            ctx_.check(glide_search_on_sub(ctx_.get(), d_part.data_handle(), dim, d_graph.data_handle(), degree_, d_map.data_handle(),
                                           start_points_[s], d_query.data_handle(), q, d_routes.data_handle(), centroids_.rows, s, &p,
                                           (int) metric_, d_ids.data_handle(), d_dists.data_handle()));
            seconds += ctx_.last_kernel_seconds();
        }
        std::printf("query time: %g s   QPS: %g\n", seconds, q / seconds);
        if (!result_file.empty()) append_result(result_file, stream_text(seconds) + "," + stream_text(q / seconds) + ",");
        result_ids = HostMatrix<uint32_t>(q, param.top_k);
        result_dists = HostMatrix<float>(q, param.top_k);
        d_ids.download(result_ids.data_handle(), result_ids.size());
        d_dists.download(result_dists.data_handle(), result_dists.size());
    }

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
};

}  // namespace glide_b200
