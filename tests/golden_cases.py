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
