// large_build: argv contract of the reference's main (large_build.cu:5-36):
//   preprocess_file knn_file graph_base_file result_file metric graph_degree knn_degree relaxant_factor
//   beam refine_beam [seed] [device]
// Writes graph_base_file.{graph,sp} (large_build.cu:94-95).
#include <iostream>
#include "../../include/glide_b200_large.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 11 || argc > 13) {
        std::cout << argv[0] << " preprocess_file knn_file graph_base_file result_file metric graph_degree knn_degree relaxant_factor beam refine_beam [seed] [device]" << std::endl;
        return -1;
    }
    try {
        const std::string preprocess_file(argv[1]), knn_file(argv[2]), graph_base_file(argv[3]), result_file(argv[4]);
        IndexParameter build_param;
        build_param.metric = parse_metric(argv[5]);
        build_param.graph_degree = (uint32_t) std::stoi(argv[6]);
        build_param.knn_degree = (uint32_t) std::stoi(argv[7]);
        build_param.relaxant_factor = std::stof(argv[8]);
        SearchParameter search_param_knn, search_param_refine;   // large_build.cu:56-81: both sized from knn_degree
        search_param_knn.beam = (uint32_t) std::stoi(argv[9]);
        derive_search_params(search_param_knn, build_param.knn_degree);
        search_param_refine.beam = (uint32_t) std::stoi(argv[10]);
        if (search_param_refine.beam != 0) derive_search_params(search_param_refine, build_param.knn_degree);
        const uint64_t seed = argc > 11 ? std::stoull(argv[11]) : 0;
        Context ctx(argc > 12 ? std::stoi(argv[12]) : 0);

        auto h_centroids = load_matrix_data<float>(preprocess_file + ".centroid");
        std::vector<uint32_t> seg_start, seg_len;
        load_segment(preprocess_file + ".segment", seg_start, seg_len);
        auto h_map = load_vector_data(preprocess_file + ".map");
        auto h_reorder = load_matrix_data<float>(preprocess_file + ".reorder");
        auto h_knn = load_matrix_data<int>(knn_file);
        if (h_knn.cols != build_param.knn_degree) throw std::invalid_argument("knn file degree differs from knn_degree");

        GLIDE_large index(ctx, build_param.graph_degree, build_param.metric, std::move(h_reorder), std::move(h_map),
                          std::move(h_centroids), std::move(seg_start), std::move(seg_len));
        append_result(result_file, stream_text(build_param.graph_degree) + ",");
        index.build(build_param, search_param_knn, search_param_refine, h_knn, result_file, seed);
        save_matrix_data(graph_base_file + ".graph", index.graph_view());
        save_vector_data(graph_base_file + ".sp", index.start_point_view());
    } catch (const std::exception &e) {
        std::cerr << "large_build: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
