// large_knn: argv contract of the reference's main (large_knn.cu:5-30):
//   preprocess_file knn_file result_file knn_degree [metric] [seed] [device]
#include <iostream>
#include "../../include/glide_b200_large.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 5 || argc > 8) {
        std::cout << argv[0] << " preprocess_file knn_file result_file knn_degree [metric] [seed] [device]" << std::endl;
        return -1;
    }
    try {
        const std::string preprocess_file(argv[1]), knn_file(argv[2]), result_file(argv[3]);
        NNDescentParameter param((size_t) std::stoi(argv[4]));
        const Metric metric = argc > 5 ? parse_metric(argv[5]) : Metric::Euclidean;
        const uint64_t seed = argc > 6 ? std::stoull(argv[6]) : 0;
        Context ctx(argc > 7 ? std::stoi(argv[7]) : 0);
        auto h_reorder = load_matrix_data<float>(preprocess_file + ".reorder");
        std::vector<uint32_t> seg_start, seg_len;
        load_segment(preprocess_file + ".segment", seg_start, seg_len);
        auto knn = build_knn_for_large(ctx, param, h_reorder, seg_start, seg_len, result_file, metric, seed);
        save_matrix_data(knn_file, knn);
    } catch (const std::exception &e) {
        std::cerr << "large_knn: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
