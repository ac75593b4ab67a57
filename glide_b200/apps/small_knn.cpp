// small_knn: argv contract of the reference's main (small_knn.cu:5-17):
//   preprocess_file knn_file result_file knn_degree [metric] [seed] [device]
#include <iostream>
#include "../../include/glide_b200.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 5 || argc > 8) {
        std::cout << argv[0] << " preprocess_file knn_file result_file knn_degree [metric] [seed] [device]" << std::endl;
        return -1;
    }
    try {
        const std::string preprocess_file(argv[1]), knn_file(argv[2]), result_file(argv[3]);
        const uint32_t knn_degree = (uint32_t) std::stoi(argv[4]);
        const Metric metric = argc > 5 ? parse_metric(argv[5]) : Metric::Euclidean;
        const uint64_t seed = argc > 6 ? std::stoull(argv[6]) : 0;
        Context ctx(argc > 7 ? std::stoi(argv[7]) : 0);
        auto h_data = load_matrix_data<float>(preprocess_file + ".reorder");
        std::vector<uint32_t> seg_start, seg_len;
        load_segment(preprocess_file + ".segment", seg_start, seg_len);
        NNDescentParameter nnd_param(knn_degree);
        DeviceBuffer<float> d_reorder(ctx, h_data.data_handle(), h_data.size());
        auto knn = build_nnd(ctx, nnd_param, d_reorder, h_data.rows, h_data.cols, seg_start, seg_len, result_file, metric, seed, true);
        save_matrix_data(knn_file, knn);
    } catch (const std::exception &e) {
        std::cerr << "small_knn: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
