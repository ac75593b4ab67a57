// large_preprocess: argv contract of the reference's main (large_preprocess.cu:5-33):
//   data_file preprocess_file result_file centroid_num sample_factor metric [seed] [device]
// Writes preprocess_file.{centroid,segment,map,reorder} (large_preprocess.cu:37-40, :77-80).
#include <iostream>
#include "../../include/glide_b200_large.hpp"
using namespace glide_b200;

int main(int argc, char **argv) {
    if (argc < 7 || argc > 9) {
        std::cout << argv[0] << " data_file preprocess_file result_file centroid_num sample_factor metric [seed] [device]" << std::endl;
        return -1;
    }
    try {
        const std::string data_file(argv[1]), preprocess_file(argv[2]), result_file(argv[3]);
        PartitionParameter param;
        param.centroid_num = (uint32_t) std::stoi(argv[4]);
        param.sample_factor = std::stof(argv[5]);
        param.metric = parse_metric(argv[6]);
        const uint64_t seed = argc > 7 ? std::stoull(argv[7]) : 0;
        Context ctx(argc > 8 ? std::stoi(argv[8]) : 0);
        // the file is read while the GPU assigns the chunks already in memory (the reference loads it
        // first, large_preprocess.cu:56, and assigns in 10 batches, :59)
        HostMatrix<float> h_data, h_reorder, h_centroids;
        std::vector<uint32_t> h_map, seg_start, seg_len;
        preprocess_for_large(ctx, param, data_file, h_data, h_reorder, h_map, seg_start, seg_len, h_centroids, result_file, seed);
        save_matrix_data(preprocess_file + ".centroid", h_centroids);
        save_segment(preprocess_file + ".segment", seg_start, seg_len);
        save_vector_data(preprocess_file + ".map", h_map);
        save_matrix_data(preprocess_file + ".reorder", h_reorder);
    } catch (const std::exception &e) {
        std::cerr << "large_preprocess: " << e.what() << std::endl;
        return 1;
    }
    return 0;
}
