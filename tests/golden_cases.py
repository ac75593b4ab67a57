"""Seeded inputs shared by tests/golden/make_reference_goldens.py (which runs the reference's kernels
on them) and tests/test_reference_goldens.py (which runs the CPU oracle on them)."""
import numpy as np

import helpers
import oracle

DEGREE = 16
BOUNDARY = 1.1
BEAMS = (32, 64, 100)
CASES = {
    "uniform32": dict(kind="uniform", n=2500, dim=32, nq=100, metric=oracle.EUCLIDEAN),
    "int128": dict(kind="int", n=2500, dim=128, nq=100, metric=oracle.EUCLIDEAN),   # exact distance ties occur
    "unit96": dict(kind="unit", n=2000, dim=96, nq=80, metric=oracle.COSINE),
}
_cache = {}


def inputs(name):
    """(base, queries, stage dict of the oracle's pipeline in the reference's summation order)."""
    if name not in _cache:
        c = CASES[name]
        base, queries = helpers.small_dataset(c["kind"], c["n"], c["dim"], c["nq"], seed=41)
        P = helpers.oracle_pipeline(base, metric=c["metric"], order=oracle.ORDER_REF, route_order=oracle.ORDER_REF,
                                    centroid_num=3)
        _cache[name] = (base, queries, P)
    return _cache[name]


def beams_full(P, base):
    """True when every build and boundary beam ends full (the reference's pruning reads unfilled slots as rows)."""
    n = base.shape[0]
    beam = P["p_build"].beam
    _, counters = oracle.build_rows(P["reorder_data"], P["knn"].view(np.uint32), P["seg_start"], P["seg_len"], P["local_sp"],
                                    P["mapping"], n, DEGREE, P["p_build"], P["alpha"], P["metric"], oracle.ORDER_REF,
                                    want_counters=True)
    sizes = np.zeros(P["reorder_data"].shape[0] - n, np.uint64)
    if sizes.size:
        g = P["after_build"].copy()
        oracle.build_boundary(P["reorder_data"], P["knn"].view(np.uint32), n, int(P["local_sp"][-1]), P["mapping"], g,
                              P["p_build"], P["alpha"], P["metric"], oracle.ORDER_REF, pool_sizes=sizes)
    return bool((counters[:, 3] == beam).all() and (sizes == beam).all())


# ---- large path: uint8-valued rows, four disjoint partitions, exact per-partition kNN lists ----
LARGE_DEGREE, LARGE_KNN = 24, 16
LARGE_ROUTES = ((1, 1.0), (2, 1.2), (3, 1.05), (4, 2.0))
LARGE_SEARCHES = ((32, 10), (64, 10), (100, 40))
_large = {}


def large_inputs():
    """Rows and queries with values in 0..255 (held as fp32 here, sent as uint8 to the reference's
    kernels), centroids, partitions, and per partition its rows, exact kNN lists, id map, start point
    and the oracle's build_for_large graph (None where a build beam stays unfilled: the reference's
    pruning would then read out of bounds, so its kernel is not run on that partition)."""
    if not _large:
        base, queries = helpers.small_dataset("int", 3000, 128, 120, seed=43)
        assert base.min() >= 0 and base.max() <= 255 and np.array_equal(base, np.rint(base))
        C = 4
        centroids, _, _ = oracle.kmeans(base[:600], C, 10, order=oracle.ORDER_REF)
        seg_index, seg_start, seg_len = oracle.define_partition(base, centroids, -1.0, order=oracle.ORDER_REF)
        rd, mapping = oracle.reorder(base, seg_index, seg_start, 0)
        o = oracle.SearchParams.derive(64, LARGE_KNN)
        one = np.array([0], np.uint32)
        parts = []
        for s in range(C):
            lo, ln = int(seg_start[s]), int(seg_len[s])
            rows = np.ascontiguousarray(rd[lo:lo + ln])
            knn = helpers.exact_partition_knn(rows, one, np.array([ln], np.uint32), LARGE_KNN, oracle.EUCLIDEAN).view(np.uint32)
            sp = (7 * s + 3) % ln
            graph, counters = oracle.build_rows(rows, knn, one, np.array([ln], np.uint32), np.array([sp], np.uint32),
                                                np.arange(ln, dtype=np.uint32), ln, LARGE_DEGREE, o, 1.05, oracle.EUCLIDEAN,
                                                oracle.ORDER_REF, want_counters=True)
            parts.append(dict(lo=lo, ln=ln, rows=rows, knn=knn, map=np.ascontiguousarray(mapping[lo:lo + ln]), sp=sp,
                              graph=graph, beams_full=bool((counters[:, 3] == o.beam).all())))
        _large.update(base=base, queries=queries, centroids=centroids, seg_index=seg_index, seg_start=seg_start,
                      seg_len=seg_len, reorder_data=rd, mapping=mapping, parts=parts, C=C, p_build=o)
    return _large
