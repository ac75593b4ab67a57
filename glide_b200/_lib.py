"""ctypes binding of ``libglide_b200.so`` (the C ABI declared in ``include/glide_b200.h``).

There is no fallback: if the library is missing or a symbol cannot be bound, importing
the product API raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# GLIDE_B200_LIB selects another build of the same library (A/B comparisons of kernel variants)
LIB_PATH = os.environ.get("GLIDE_B200_LIB") or os.path.join(_HERE, "libglide_b200.so")

u32, u64, i32, f32, vp = C.c_uint32, C.c_uint64, C.c_int, C.c_float, C.c_void_p
P = C.POINTER


class SearchParamsC(C.Structure):
    _fields_ = [("top_k", u32), ("beam", u32), ("max_iterations", u32), ("min_iterations", u32),
                ("hash_bit", u32), ("hash_reset_interval", u32)]


# name -> (restype, argtypes); mirrors include/glide_b200.h one to one
SIGNATURES = {
    "glide_ctx_create": (i32, [i32, P(vp)]),
    "glide_ctx_destroy": (None, [vp]),
    "glide_last_error": (C.c_char_p, [vp]),
    "glide_ctx_stream": (vp, [vp]),
    "glide_last_kernel_ms": (f32, [vp]),
    "glide_ctx_workspace_bytes": (C.c_size_t, [vp]),
    "glide_calculate_hash_bitlen": (u32, [u32, u32, f32, u32]),
    "glide_calculate_hash_reset_interval": (u32, [u32, u32, f32, u32]),
    "glide_adjust_search_params": (None, [u32, P(u32), P(u32)]),
    "glide_get_centroids": (i32, [vp, vp, u32, u32, u32, f32, u64, u32, i32, vp, P(u32)]),
    "glide_sample_ids": (i32, [u32, u32, u64, vp]),
    "glide_kmeans_fit": (i32, [vp, vp, u32, u32, u32, u32, i32, i32, vp, vp, P(u32)]),
    "glide_define_partition": (i32, [vp, vp, u32, u32, vp, u32, f32, i32, vp, vp, vp]),
    "glide_reorder": (i32, [vp, vp, u32, u32, vp, vp, u32, vp, vp]),
    "glide_preprocess": (i32, [vp, vp, u32, u32, u32, f32, f32, i32, u64, vp, vp, vp, P(vp), P(vp), P(u32)]),
    "glide_free": (None, [vp]),
    "glide_build_nnd": (i32, [vp, vp, u32, u32, vp, vp, u32, u32, u32, f32, u32, u32, u64, i32, vp, P(u32)]),
    "glide_bruteforce_knn": (i32, [vp, vp, u32, vp, u32, u32, u32, i32, vp, vp]),
    "glide_start_point_select": (i32, [vp, vp, u32, vp, u64, vp, vp]),
    "glide_subgraph_build_and_merge": (i32, [vp, vp, u32, u32, vp, u32, vp, vp, u32, vp, vp, u32, u32,
                                             P(SearchParamsC), f32, i32, i32, vp]),
    "glide_subgraph_build_range": (i32, [vp, vp, u32, u32, vp, u32, vp, vp, u32, vp, vp, u32, u32,
                                         P(SearchParamsC), f32, i32, u32, u32, vp]),
    "glide_reverse_graph": (i32, [vp, vp, u32, u32]),
    "glide_refine_rows": (i32, [vp, vp, u32, u32, vp, u32, vp, u32, vp, P(SearchParamsC), f32, i32, u32, u32, vp]),
    "glide_subgraph_build_rows": (i32, [vp, vp, u32, u32, vp, u32, vp, vp, u32, vp, vp, u32, u32,
                                        P(SearchParamsC), f32, i32, u32, u32, vp]),
    "glide_build_nnd_range": (i32, [vp, vp, u32, u32, vp, vp, u32, u32, u32, f32, u32, u32, u64, i32, u32, vp, P(u32)]),
    "glide_comm_unique_id": (i32, [vp]),
    "glide_comm_init": (i32, [vp, vp, u32, u32]),
    "glide_comm_destroy": (i32, [vp]),
    "glide_comm_world": (u32, [vp]),
    "glide_comm_rank": (u32, [vp]),
    "glide_comm_all_gather_v": (i32, [vp, vp, vp, vp]),
    "glide_comm_broadcast": (i32, [vp, vp, u64, u32]),
    "glide_comm_all_reduce_u64": (i32, [vp, vp, u64, i32]),
    "glide_ctx_synchronize": (i32, [vp]),
    "glide_refine": (i32, [vp, vp, u32, u32, vp, u32, vp, u32, vp, P(SearchParamsC), f32, i32]),
    "glide_refine_waves": (i32, [vp, vp, u32, u32, vp, u32, vp, u32, vp, P(SearchParamsC), f32, i32, u32]),
    "glide_search": (i32, [vp, vp, u32, u32, vp, u32, vp, u32, vp, vp, u32, P(SearchParamsC), i32, vp, vp]),
    "glide_search_host": (i32, [vp, vp, u32, u32, vp, u32, vp, u32, vp, vp, u32, P(SearchParamsC), i32, vp, vp]),
    "glide_tc_knn_fallbacks": (u32, [vp]),
    "glide_matrix_file_info": (i32, [C.c_char_p, u32, P(u32), P(u32)]),
    "glide_load_rows": (i32, [vp, C.c_char_p, u32, u64, u64, vp, u32, u32, vp, u32, i32, vp, P(C.c_double)]),
    "glide_search_pipe_create": (i32, [vp, u32, u32, u32, u32, P(vp)]),
    "glide_search_pipe_destroy": (None, [vp]),
    "glide_search_pipe_submit": (i32, [vp, vp, u32, u32, vp, u32, vp, u32, vp, vp, u32, P(SearchParamsC), i32, vp, vp, P(u32)]),
    "glide_search_pipe_wait": (i32, [vp, u32]),
    "glide_search_static_scratch": (i32, [vp, vp, u32, u32, vp, u32, vp, u32, vp, vp, u32, P(SearchParamsC), i32, vp, vp]),
    "glide_last_search_split_ms": (None, [vp, P(f32)]),
    "glide_last_search_launches": (u32, [vp]),
    "glide_enable_counters": (None, [vp, i32]),
    "glide_read_counters": (i32, [vp, P(u64)]),
    "glide_select_segments": (i32, [vp, vp, u32, u32, vp, u32, u32, f32, i32, vp]),
    "glide_search_on_sub": (i32, [vp, vp, u32, vp, u32, vp, u32, vp, u32, vp, u32, u32, P(SearchParamsC), i32,
                                  vp, vp]),
    "glide_build_partition": (i32, [vp, vp, u32, u32, vp, u32, u32, u32, P(SearchParamsC), f32, i32, vp]),
    "glide_refine_partition": (i32, [vp, vp, u32, u32, vp, u32, u32, P(SearchParamsC), f32, i32]),
    "glide_host_alloc": (i32, [C.c_size_t, P(vp)]),
    "glide_host_free": (None, [vp]),
    "glide_host_register": (i32, [vp, C.c_size_t]),
    "glide_host_unregister": (i32, [vp]),
    "glide_large_create": (i32, [vp, vp, i32, u32, vp, vp, u32, vp, u32, i32, vp, P(vp)]),
    "glide_large_destroy": (None, [vp]),
    "glide_large_set_start_points": (i32, [vp, vp]),
    "glide_large_get_start_points": (i32, [vp, vp]),
    "glide_large_build": (i32, [vp, vp, u32, u32, P(SearchParamsC), P(SearchParamsC), f32, u32, f32, u32, u32, u64, vp, vp]),
    "glide_large_make_resident": (i32, [vp, vp, u32, C.c_size_t, P(u32)]),
    "glide_large_search": (i32, [vp, vp, u32, vp, u32, u32, f32, P(SearchParamsC), vp, u32, vp, vp]),
    "glide_large_last_stats": (None, [vp, P(C.c_double)]),
    "glide_large_resident_buffers": (i32, [vp, u32, P(vp), P(vp), P(vp)]),
    "glide_large_merge": (i32, [vp, vp, u32, f32, u32, P(SearchParamsC), P(C.c_double)]),
    "glide_large_search_merged": (i32, [vp, vp, u32, vp, u32, P(SearchParamsC), vp, vp]),
    "glide_large_merged_graph": (i32, [vp, vp]),
    "glide_merge_results": (i32, [vp, vp, vp, u32, u32, u32, vp, vp]),
    "glide_malloc": (i32, [vp, C.c_size_t, P(vp)]),
    "glide_memcpy_h2d": (i32, [vp, vp, vp, C.c_size_t]),
    "glide_memcpy_d2h": (i32, [vp, vp, vp, C.c_size_t]),
    "glide_memset_u32": (i32, [vp, vp, u32, C.c_size_t]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `make -C glide_b200/csrc` (or __graft_entry__.build()). "
            "glide_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
