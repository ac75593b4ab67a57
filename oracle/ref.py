"""ctypes front end of oracle/_ref/libglide_ref.so: the REFERENCE's own kernels behind the
harness in ref_harness.cu. TEST INFRASTRUCTURE, used only by the GPU tests that pin the CPU
oracle against the reference; absent when the reference tree was not available at build time."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libglide_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
    return _lib


u32, f32, i32, vp = C.c_uint32, C.c_float, C.c_int, C.c_void_p


def search(d_data, dim, d_graph, degree, d_centroids, c, d_sp, d_queries, q, p, metric, d_ids, d_dists) -> int:
    return lib().ref_search(vp(d_data), u32(dim), vp(d_graph), u32(degree), vp(d_centroids), u32(c), vp(d_sp), vp(d_queries),
                            u32(q), u32(p.top_k), u32(p.beam), u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                            u32(p.hash_reset_interval), i32(metric), vp(d_ids), vp(d_dists))


def build(d_reorder, reorder_num, dim, d_knn, knn_degree, d_seg_start, d_seg_len, segment_num, d_local_sp, d_map, num,
          graph_degree, p, alpha, metric, with_boundary, d_graph) -> int:
    return lib().ref_build(vp(d_reorder), u32(reorder_num), u32(dim), vp(d_knn), u32(knn_degree), vp(d_seg_start),
                           vp(d_seg_len), u32(segment_num), vp(d_local_sp), vp(d_map), u32(num), u32(graph_degree), u32(p.beam),
                           u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit), u32(p.hash_reset_interval),
                           f32(alpha), i32(metric), i32(1 if with_boundary else 0), vp(d_graph))


def reverse(d_graph, num, degree) -> int:
    return lib().ref_reverse(vp(d_graph), u32(num), u32(degree))


def refine(d_data, num, dim, d_graph, degree, d_centroids, c, d_sp, p, alpha, metric) -> int:
    return lib().ref_refine(vp(d_data), u32(num), u32(dim), vp(d_graph), u32(degree), vp(d_centroids), u32(c), vp(d_sp),
                            u32(p.beam), u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                            u32(p.hash_reset_interval), f32(alpha), i32(metric))


def define_partition(d_data, num, dim, d_centroids, c, boundary_factor, metric, d_seg_len, d_seg_index) -> int:
    return lib().ref_define_partition(vp(d_data), u32(num), u32(dim), vp(d_centroids), u32(c), f32(boundary_factor),
                                      i32(metric), vp(d_seg_len), vp(d_seg_index))


def reorder(d_data, d_reorder, d_seg_index, d_map, d_seg_start, num, dim) -> int:
    return lib().ref_reorder(vp(d_data), vp(d_reorder), vp(d_seg_index), vp(d_map), vp(d_seg_start), u32(num), u32(dim))


# ---- large path (uint8 rows and queries, as the reference instantiates it) ----
def define_partition_for_large(d_data_u8, batch_size, dim, d_centroids, c, metric, d_seg_len, d_seg_index) -> int:
    return lib().ref_define_partition_for_large(vp(d_data_u8), u32(batch_size), u32(dim), vp(d_centroids), u32(c), i32(metric),
                                                vp(d_seg_len), vp(d_seg_index))


def build_for_large(d_data_u8, length, dim, d_knn, knn_degree, start_point, graph_degree, p, alpha, metric, d_graph) -> int:
    return lib().ref_build_for_large(vp(d_data_u8), u32(length), u32(dim), vp(d_knn), u32(knn_degree), u32(start_point),
                                     u32(graph_degree), u32(p.beam), u32(p.max_iterations), u32(p.min_iterations),
                                     u32(p.hash_bit), u32(p.hash_reset_interval), f32(alpha), i32(metric), vp(d_graph))


def refine_for_large(d_data_u8, length, dim, d_graph, graph_degree, start_point, p, alpha, metric) -> int:
    return lib().ref_refine_for_large(vp(d_data_u8), u32(length), u32(dim), vp(d_graph), u32(graph_degree), u32(start_point),
                                      u32(p.beam), u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                                      u32(p.hash_reset_interval), f32(alpha), i32(metric))


def select_segments(d_queries_u8, q, dim, d_centroids, c, min_segment_num, boundary_factor, metric, d_segment_ids) -> int:
    return lib().ref_select_segments(vp(d_queries_u8), u32(q), u32(dim), vp(d_centroids), u32(c), u32(min_segment_num),
                                     f32(boundary_factor), i32(metric), vp(d_segment_ids))


def search_on_sub(d_data_u8, dim, d_graph, graph_degree, d_map, start_point, d_queries_u8, q, d_segment_ids, segment_num,
                  segment_id, p, metric, d_final_ids, d_final_dists) -> int:
    return lib().ref_search_on_sub(vp(d_data_u8), u32(dim), vp(d_graph), u32(graph_degree), vp(d_map), u32(start_point),
                                   vp(d_queries_u8), u32(q), vp(d_segment_ids), u32(segment_num), u32(segment_id),
                                   u32(p.top_k), u32(p.beam), u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                                   u32(p.hash_reset_interval), i32(metric), vp(d_final_ids), vp(d_final_dists))


def last_seconds() -> float:
    """Device time of the kernels of the last harness call (CUDA events)."""
    f = lib().ref_last_ms
    f.restype = C.c_float
    return float(f()) / 1000.0
