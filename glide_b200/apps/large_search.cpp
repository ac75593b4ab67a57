// large_search: argv contract of the reference's main (large_search.cu:38-69):
//   preprocess_file query_file truth_file graph_base_file result_file metric topk search_beam
//   min_graph_num boundary_factor [device]
#include <iostream>
#include "../../include/glide_b200_large.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 11 || argc > 12) {
        std::cout << argv[0] << " preprocess_file query_file truth_file graph_base_file result_file metric topk search_beam min_graph_num boundary_factor [device]" << std::endl;
        return -1;
    }
    try {
        const std::string preprocess_file(argv[1]), query_file(argv[2]), truth_file(argv[3]), graph_base_file(argv[4]), result_file(argv[5]);
        const Metric metric = parse_metric(argv[6]);
        SearchParameter search_param;
        search_param.top_k = (uint32_t) std::stoi(argv[7]);
        search_param.beam = (uint32_t) std::stoi(argv[8]);
        const uint32_t min_segment_num = (uint32_t) std::stoi(argv[9]);
        const float boundary_factor = std::stof(argv[10]);
        Context ctx(argc > 11 ? std::stoi(argv[11]) : 0);

        auto h_centroids = load_matrix_data<float>(preprocess_file + ".centroid");
        std::vector<uint32_t> seg_start, seg_len;
        load_segment(preprocess_file + ".segment", seg_start, seg_len);
        auto h_map = load_vector_data(preprocess_file + ".map");
        auto h_reorder = load_matrix_data<float>(preprocess_file + ".reorder");
        auto query = load_matrix_data<float>(query_file);
        auto truth = load_matrix_data<uint32_t>(truth_file);
        auto graph = load_matrix_data<uint32_t>(graph_base_file + ".graph");
        auto start_point = load_vector_data(graph_base_file + ".sp");

        append_result(result_file, stream_text(search_param.beam) + ",");
        derive_search_params(search_param, graph.cols);   // large_search.cu:98-110
        GLIDE_large index(ctx, graph.cols, metric, std::move(h_reorder), std::move(h_map), std::move(h_centroids),
                          std::move(seg_start), std::move(seg_len));
        index.load(graph, start_point);
        HostMatrix<uint32_t> result_ids;
        HostMatrix<float> result_dists;
        index.search(search_param, min_segment_num, boundary_factor, query, result_ids, result_dists, result_file);
        const float recall = calculate_recall(result_ids, truth, search_param.top_k);
        append_result(result_file, stream_text(recall) + "\n");
    } catch (const std::exception &e) {
        std::cerr << "large_search: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
