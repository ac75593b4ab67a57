// small_search: argv contract of the reference's main (small_search.cu:38-55):
//   data_file query_file truth_file preprocess_file graph_base_file result_file metric topk search_beam [device]
#include <iostream>
#include "../../include/glide_b200.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 10 || argc > 11) {
        std::cout << argv[0] << " data_file query_file truth_file preprocess_file graph_base_file result_file metric topk search_beam [device]" << std::endl;
        return -1;
    }
    try {
        const std::string data_file(argv[1]), query_file(argv[2]), truth_file(argv[3]), preprocess_file(argv[4]), graph_base_file(argv[5]), result_file(argv[6]);
        const Metric metric = parse_metric(argv[7]);
        Context ctx(argc > 10 ? std::stoi(argv[10]) : 0);
        auto data = load_matrix_data<float>(data_file);
        auto query = load_matrix_data<float>(query_file);
        auto truth = load_matrix_data<uint32_t>(truth_file);
        auto graph = load_matrix_data<uint32_t>(graph_base_file + ".graph");
        auto start_point = load_vector_data(graph_base_file + ".sp");
        auto centroids = load_matrix_data<float>(preprocess_file + ".centroid");
        SearchParameter search_param;
        search_param.top_k = (uint32_t) std::stoi(argv[8]);
        search_param.beam = (uint32_t) std::stoi(argv[9]);
        append_result(result_file, stream_text(search_param.beam) + ",");
        derive_search_params(search_param, graph.cols);   // small_search.cu:98-107
        GLIDE index(ctx, graph.cols, data, centroids, metric);
        index.load(graph, start_point);
        HostMatrix<uint32_t> result_ids;
        HostMatrix<float> result_dists;
        index.search(search_param, query, result_ids, result_dists, result_file);
        const float recall = calculate_recall(result_ids, truth, search_param.top_k);
        append_result(result_file, stream_text(recall) + "\n");
    } catch (const std::exception &e) {
        std::cerr << "small_search: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
