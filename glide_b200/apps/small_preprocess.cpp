// small_preprocess: argv contract of the reference's main (small_preprocess.cu:6-21):
//   data_file preprocess_file result_file centroid_num boundary_factor sample_factor metric [seed] [device]
// Writes <preprocess_file>.centroid/.segment/.map/.reorder and the CSV header + preprocess time.
#include <iostream>
#include "../../include/glide_b200.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 8 || argc > 10) {
        std::cout << argv[0] << " data_file preprocess_file result_file centroid_num boundary_factor sample_factor metric [seed] [device]" << std::endl;
        return -1;
    }
    try {
        const std::string data_file(argv[1]), preprocess_file(argv[2]), result_file(argv[3]);
        PartitionParameter param;
        param.centroid_num = (uint32_t) std::stoi(argv[4]);
        param.boundary_factor = std::stof(argv[5]);
        param.sample_factor = std::stof(argv[6]);
        param.metric = parse_metric(argv[7]);
        const uint64_t seed = argc > 8 ? std::stoull(argv[8]) : 0;
        Context ctx(argc > 9 ? std::stoi(argv[9]) : 0);
        append_result(result_file, "pre_time,knn_time,degree,index_time,beam,search_time,QPS,recall\n");  // small_preprocess.cu:54-56
        auto h_data = load_matrix_data<float>(data_file);
        DeviceBuffer<float> d_data(ctx, h_data.data_handle(), h_data.size());
        DeviceBuffer<float> d_reorder, d_centroids;
        DeviceBuffer<uint32_t> d_map;
        std::vector<uint32_t> seg_start, seg_len;
        uint32_t reorder_num = 0;
        preprocess(ctx, param, d_data, h_data.rows, h_data.cols, d_reorder, d_map, seg_start, seg_len, d_centroids,
                   reorder_num, result_file, seed);
        HostMatrix<float> h_centroids(param.centroid_num, h_data.cols), h_reorder(reorder_num, h_data.cols);
        std::vector<uint32_t> h_map(reorder_num);
        d_centroids.download(h_centroids.data_handle(), h_centroids.size());
        d_reorder.download(h_reorder.data_handle(), h_reorder.size());
        d_map.download(h_map.data(), h_map.size());
        save_matrix_data(preprocess_file + ".centroid", h_centroids);
        save_segment(preprocess_file + ".segment", seg_start, seg_len);
        save_vector_data(preprocess_file + ".map", h_map);
        save_matrix_data(preprocess_file + ".reorder", h_reorder);
    } catch (const std::exception &e) {
        std::cerr << "small_preprocess: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
