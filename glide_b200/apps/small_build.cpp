// small_build: argv contract of the reference's main (small_build.cu:5-24):
//   data_file preprocess_file knn_file graph_base_file result_file metric graph_degree knn_degree
//   relaxant_factor beam refine_beam [seed] [device]
#include <iostream>
#include "../../include/glide_b200.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 12 || argc > 14) {
        std::cout << argv[0] << " data_file preprocess_file knn_file graph_base_file result_file metric graph_degree knn_degree relaxant_factor beam refine_beam [seed] [device]" << std::endl;
        return -1;
    }
    try {
        const std::string data_file(argv[1]), preprocess_file(argv[2]), knn_file(argv[3]), graph_base_file(argv[4]), result_file(argv[5]);
        IndexParameter build_param;
        build_param.metric = parse_metric(argv[6]);
        build_param.graph_degree = (uint32_t) std::stoi(argv[7]);
        build_param.knn_degree = (uint32_t) std::stoi(argv[8]);
        build_param.relaxant_factor = std::stof(argv[9]);
        SearchParameter search_param_knn, search_param_refine;   // small_build.cu:61-82: both sized from knn_degree
        search_param_knn.beam = (uint32_t) std::stoi(argv[10]);
        derive_search_params(search_param_knn, build_param.knn_degree);
        search_param_refine.beam = (uint32_t) std::stoi(argv[11]);
        if (search_param_refine.beam != 0) derive_search_params(search_param_refine, build_param.knn_degree);
        const uint64_t seed = argc > 12 ? std::stoull(argv[12]) : 0;
        Context ctx(argc > 13 ? std::stoi(argv[13]) : 0);

        auto h_data = load_matrix_data<float>(data_file);
        auto h_centroids = load_matrix_data<float>(preprocess_file + ".centroid");
        std::vector<uint32_t> seg_start, seg_len;
        load_segment(preprocess_file + ".segment", seg_start, seg_len);
        auto h_map = load_vector_data(preprocess_file + ".map");
        auto h_reorder = load_matrix_data<float>(preprocess_file + ".reorder");
        auto h_knn = load_matrix_data<int>(knn_file);
        if (h_knn.cols != build_param.knn_degree) throw std::invalid_argument("knn file degree differs from knn_degree");

        DeviceBuffer<float> d_reorder(ctx, h_reorder.data_handle(), h_reorder.size());
        DeviceBuffer<uint32_t> d_map(ctx, h_map.data(), h_map.size());
        DeviceBuffer<int> d_knn(ctx, h_knn.data_handle(), h_knn.size());
        GLIDE index(ctx, build_param.graph_degree, h_data, h_centroids, build_param.metric);
        append_result(result_file, stream_text(build_param.graph_degree) + ",");
        index.build(build_param, search_param_knn, search_param_refine, d_knn, seg_start, seg_len, d_map, h_map, d_reorder,
                    h_reorder.rows, result_file, seed);

        HostMatrix<uint32_t> graph(index.num(), index.graph_degree());
        index.graph_view().download(graph.data_handle(), graph.size());
        std::vector<uint32_t> sp(index.start_point_num());
        index.start_point_view().download(sp.data(), sp.size());
        save_matrix_data(graph_base_file + ".graph", graph);
        save_vector_data(graph_base_file + ".sp", sp);
    } catch (const std::exception &e) {
        std::cerr << "small_build: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
