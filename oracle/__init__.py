"""ctypes/numpy front end of the CPU oracle (``glide_oracle.cpp``).

TEST INFRASTRUCTURE: only tests, the smoke check and the benchmark's CPU-baseline
leg may import this package. The product package never does.

Pinned on the GPU against the reference's own kernels (``ref_harness.cu``,
``tests/test_gpu_reference.py``) for search, build, boundary merge, reverse edges, refine and
assignment; PARITY UNPINNED for k-means and NN-descent (cuVS arithmetic, not in the reference
tree). See the header of ``glide_oracle.cpp``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libglide_oracle.so")

EUCLIDEAN, COSINE = 0, 1
# ORDER_WARP: candidate scoring / pruning order of the CUDA kernels; ORDER_TEAM: their order for
# centroid distances (routing, assignment, k-means); ORDER_REF: the reference's own.
ORDER_REF, ORDER_TEAM, ORDER_WARP = 0, 1, 2
INVALID = 0xFFFFFFFF


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile next to this file."""
    src = os.path.join(_HERE, "glide_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_distance.restype = C.c_float
        _lib.orc_recall.restype = C.c_float
        for name in ("orc_hash_bitlen", "orc_hash_reset_interval"):
            getattr(_lib, name).restype = C.c_uint32
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


u32, f32, i32 = C.c_uint32, C.c_float, C.c_int


@dataclass
class SearchParams:
    """Derived search parameters (params.cuh:37-47, :82-99 and the callers
    small_build.cu:61-82, small_search.cu:98-107)."""
    beam: int
    max_iterations: int
    min_iterations: int
    hash_bit: int
    hash_reset_interval: int
    top_k: int = 10

    @staticmethod
    def derive(beam: int, degree_for_hash: int, top_k: int = 10, min_iterations: int = 0,
               max_iterations: int = 0, max_fill: float = 0.5, min_bitlen: int = 0) -> "SearchParams":
        b = u32(beam)
        m = u32(max_iterations)
        lib().orc_adjust_search_params(u32(min_iterations), C.byref(m), C.byref(b))
        bits = lib().orc_hash_bitlen(b, u32(degree_for_hash), f32(max_fill), u32(min_bitlen))
        interval = lib().orc_hash_reset_interval(b, u32(degree_for_hash), f32(max_fill), u32(bits))
        return SearchParams(b.value, m.value, min_iterations, bits, interval, top_k)


def distance(a, b, metric=EUCLIDEAN, order=ORDER_REF) -> float:
    a, b = _f32(a), _f32(b)
    return float(lib().orc_distance(_p(a), _p(b), u32(a.size), i32(metric), i32(order)))


def warp_sort(keys, vals, n_regs: int):
    """keys/vals laid out [lane*N + i]; returns sorted copies in the same layout."""
    k, v = _f32(keys).copy(), _u32(vals).copy()
    assert k.size == 32 * n_regs
    lib().orc_warp_sort(_p(k), _p(v), u32(n_regs))
    return k, v


def sort_with_key_value(max_number: int, vals, keys):
    k, v = _f32(keys).copy(), _u32(vals).copy()
    lib().orc_sort_with_key_value(u32(max_number), u32(k.size), _p(v), _p(k))
    return v, k


def search(data, graph, centroids, start_points, queries, p: SearchParams, metric=EUCLIDEAN,
           order=ORDER_WARP, threads=0, want_counters=False, route_order=None):
    if route_order is None:
        route_order = ORDER_REF if order == ORDER_REF else ORDER_TEAM
    data, queries, centroids = _f32(data), _f32(queries), _f32(centroids)
    graph, start_points = _u32(graph), _u32(start_points)
    Q, dim = queries.shape
    ids = np.empty((Q, p.top_k), np.uint32)
    dists = np.empty((Q, p.top_k), np.float32)
    counters = np.zeros((Q, 2), np.uint64) if want_counters else None
    rc = lib().orc_search(_p(data), u32(dim), _p(graph), u32(graph.shape[1]), _p(centroids),
                          u32(centroids.shape[0]), _p(start_points), _p(queries), u32(Q), u32(p.top_k),
                          u32(p.beam), u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                          u32(p.hash_reset_interval), i32(metric), i32(order), i32(route_order), _p(ids),
                          _p(dists), _p(counters), i32(threads))
    if rc != 0:
        raise ValueError("orc_search: unsupported shape")
    return (ids, dists, counters) if want_counters else (ids, dists)


def build_rows(reorder_data, knn, seg_start, seg_len, start_points_local, mapping, num, graph_degree,
               p: SearchParams, alpha, metric=EUCLIDEAN, order=ORDER_WARP, graph=None, first=0, count=None,
               threads=0, want_counters=False):
    reorder_data, knn = _f32(reorder_data), _u32(knn)
    seg_start, seg_len = _u32(seg_start), _u32(seg_len)
    start_points_local, mapping = _u32(start_points_local), _u32(mapping)
    if graph is None:
        graph = np.full((num, graph_degree), INVALID, np.uint32)
    count = num - first if count is None else count
    counters = np.zeros((count, 4), np.uint64) if want_counters else None
    rc = lib().orc_build_rows(_p(reorder_data), u32(reorder_data.shape[1]), _p(knn), u32(knn.shape[1]),
                              _p(seg_start), _p(seg_len), u32(seg_start.size), _p(start_points_local),
                              _p(mapping), u32(first), u32(count), u32(graph_degree), u32(p.beam),
                              u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                              u32(p.hash_reset_interval), f32(alpha), i32(metric), i32(order), _p(graph),
                              _p(counters), i32(threads))
    if rc != 0:
        raise ValueError("orc_build_rows: unsupported shape")
    return (graph, counters) if want_counters else graph


def build_boundary(reorder_data, knn, num, start_point_local, mapping, graph, p: SearchParams, alpha,
                   metric=EUCLIDEAN, order=ORDER_WARP, threads=0, pool_sizes=None):
    reorder_data, knn, mapping = _f32(reorder_data), _u32(knn), _u32(mapping)
    assert graph.dtype == np.uint32 and graph.flags.c_contiguous
    boundary_num = reorder_data.shape[0] - num
    rc = lib().orc_build_boundary(_p(reorder_data), u32(reorder_data.shape[1]), _p(knn), u32(knn.shape[1]),
                                  u32(num), u32(boundary_num), u32(start_point_local), _p(mapping),
                                  u32(graph.shape[1]), u32(p.beam), u32(p.max_iterations),
                                  u32(p.min_iterations), u32(p.hash_bit), u32(p.hash_reset_interval),
                                  f32(alpha), i32(metric), i32(order), _p(graph), _p(pool_sizes), i32(threads))
    if rc != 0:
        raise ValueError("orc_build_boundary: unsupported shape")
    return graph


def reverse_graph(graph):
    assert graph.dtype == np.uint32 and graph.flags.c_contiguous
    lib().orc_reverse_graph(_p(graph), u32(graph.shape[0]), u32(graph.shape[1]))
    return graph


def refine(data, graph_in, centroids, start_points, p: SearchParams, alpha, metric=EUCLIDEAN,
           order=ORDER_WARP, threads=0, route_order=None, pool_sizes=None, wave_rows=0):
    """wave_rows: points are refined in waves of that many consecutive ids, each wave reading the rows
    the earlier waves wrote (0: a single wave, i.e. every search reads the graph as it was before).
    centroids=None: the large path's variant (one partition, seeded from start_points[0]'s row)."""
    if route_order is None:
        route_order = ORDER_REF if order == ORDER_REF else ORDER_TEAM
    data = _f32(data)
    row_mode = centroids is None
    if not row_mode:
        centroids = _f32(centroids)
    graph_in, start_points = _u32(graph_in), _u32(np.atleast_1d(start_points))
    out = np.empty_like(graph_in)
    rc = lib().orc_refine(_p(data), u32(data.shape[0]), u32(data.shape[1]), _p(graph_in), _p(out),
                          u32(graph_in.shape[1]), _p(centroids), u32(1 if row_mode else centroids.shape[0]),
                          _p(start_points), u32(p.beam), u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                          u32(p.hash_reset_interval), f32(alpha), i32(metric), i32(order), i32(route_order),
                          _p(pool_sizes), i32(threads), u32(wave_rows), i32(1 if row_mode else 0))
    if rc != 0:
        raise ValueError("orc_refine: unsupported shape")
    return out


def define_partition(data, centroids, boundary_factor, metric=EUCLIDEAN, order=ORDER_TEAM, want_ratio=False):
    data, centroids = _f32(data), _f32(centroids)
    n, dim = data.shape
    c = centroids.shape[0]
    seg_index = np.empty((n, 3), np.uint32)
    seg_len = np.zeros(c + 1, np.uint32)
    ratio = np.empty(n, np.float32) if want_ratio else None
    lib().orc_define_partition(_p(data), u32(n), u32(dim), _p(centroids), u32(c), f32(boundary_factor),
                               i32(metric), i32(order), _p(seg_index), _p(seg_len), _p(ratio))
    seg_start = np.zeros(c + 1, np.uint32)
    seg_start[1:] = np.cumsum(seg_len[:-1], dtype=np.uint64).astype(np.uint32)  # partition.cuh:111-115
    return (seg_index, seg_start, seg_len, ratio) if want_ratio else (seg_index, seg_start, seg_len)


def reorder(data, seg_index, seg_start, boundary_num):
    data, seg_index, seg_start = _f32(data), _u32(seg_index), _u32(seg_start)
    n, dim = data.shape
    out = np.empty((n + boundary_num, dim), np.float32)
    mapping = np.empty(n + boundary_num, np.uint32)
    lib().orc_reorder(_p(data), u32(n), u32(dim), _p(seg_index), _p(seg_start), _p(out), _p(mapping))
    return out, mapping


def select_segments(queries, centroids, min_segment_num, boundary_factor, metric=EUCLIDEAN, order=ORDER_TEAM):
    queries, centroids = _f32(queries), _f32(centroids)
    out = np.empty((queries.shape[0], centroids.shape[0]), np.uint32)
    lib().orc_select_segments(_p(queries), u32(queries.shape[0]), u32(queries.shape[1]), _p(centroids),
                              u32(centroids.shape[0]), u32(min_segment_num), f32(boundary_factor),
                              i32(metric), i32(order), _p(out))
    return out


def search_on_sub(data, graph, mapping, start_point, queries, segment_ids, segment_id, p: SearchParams,
                  final_ids, final_dists, metric=EUCLIDEAN, order=ORDER_WARP, threads=0):
    data, queries = _f32(data), _f32(queries)
    graph, mapping, segment_ids = _u32(graph), _u32(mapping), _u32(segment_ids)
    assert final_ids.dtype == np.uint32 and final_dists.dtype == np.float32
    rc = lib().orc_search_on_sub(_p(data), u32(data.shape[1]), _p(graph), u32(graph.shape[1]), _p(mapping),
                                 u32(start_point), _p(queries), u32(queries.shape[0]), _p(segment_ids),
                                 u32(segment_ids.shape[1]), u32(segment_id), u32(p.top_k), u32(p.beam),
                                 u32(p.max_iterations), u32(p.min_iterations), u32(p.hash_bit),
                                 u32(p.hash_reset_interval), i32(metric), i32(order), _p(final_ids),
                                 _p(final_dists), i32(threads))
    if rc != 0:
        raise ValueError("orc_search_on_sub: unsupported shape")


def merge_results(ids, dists):
    """result_merge over whole result sets: ids, dists of shape (G, Q, top_k), folded in set order."""
    ids, dists = _u32(ids), _f32(dists)
    g, q, k = ids.shape
    out_ids, out_d = np.empty((q, k), np.uint32), np.empty((q, k), np.float32)
    if lib().orc_merge_results(_p(ids), _p(dists), u32(g), u32(q), u32(k), _p(out_ids), _p(out_d)) != 0:
        raise ValueError("orc_merge_results: unsupported shape")
    return out_ids, out_d


def load_matrix_rowwise(path: str, dtype=np.float32) -> np.ndarray:
    """The reference's loader (load.cuh:10-30): one read per row into pageable memory."""
    dtype = np.dtype(dtype)
    rows, dim = C.c_uint32(), C.c_uint32()
    if lib().orc_load_matrix_rowwise(str(path).encode(), u32(dtype.itemsize), None, C.byref(rows), C.byref(dim)) != 0:
        raise IOError(f"{path}: cannot read the header")
    out = np.empty((rows.value, dim.value), dtype)
    if lib().orc_load_matrix_rowwise(str(path).encode(), u32(dtype.itemsize), _p(out), None, None) != 0:
        raise IOError(f"{path}: ends before its last row")
    return out


def set_two_warps(on: bool) -> None:
    """Tests only: False makes the search use the single-warp sort and merge at every size."""
    lib().orc_set_two_warps(C.c_int(1 if on else 0))


def recall(neighbors, truth, top_k) -> float:
    neighbors, truth = _u32(neighbors), _u32(truth)
    return float(lib().orc_recall(_p(neighbors), u32(neighbors.shape[1]), _p(truth), u32(truth.shape[1]),
                                  u32(neighbors.shape[0]), u32(top_k)))


def bruteforce_knn(base, queries, k, metric=EUCLIDEAN, threads=0, want_dists=True):
    base, queries = _f32(base), _f32(queries)
    ids = np.empty((queries.shape[0], k), np.uint32)
    dists = np.empty((queries.shape[0], k), np.float32) if want_dists else None
    rc = lib().orc_bruteforce_knn(_p(base), u32(base.shape[0]), _p(queries), u32(queries.shape[0]),
                                  u32(base.shape[1]), u32(k), i32(metric), _p(ids), _p(dists), i32(threads))
    if rc != 0:
        raise ValueError("orc_bruteforce_knn: bad k")
    return (ids, dists) if want_dists else ids


def kmeans(sample, c, max_iter=25, order=ORDER_TEAM, metric=EUCLIDEAN, init=1):
    sample = _f32(sample)
    cent = np.empty((c, sample.shape[1]), np.float32)
    labels = np.empty(sample.shape[0], np.uint32)
    rounds = lib().orc_kmeans(_p(sample), u32(sample.shape[0]), u32(sample.shape[1]), u32(c), u32(max_iter),
                              i32(metric), i32(order), i32(init), _p(cent), _p(labels))
    if rounds < 0:
        raise ValueError("orc_kmeans: fewer rows than centroids")
    return cent, labels, rounds


def max_threads() -> int:
    return int(lib().orc_max_threads())
