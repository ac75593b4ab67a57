"""Small seeded pipelines built with the CPU oracle, shared by the CPU and GPU tests."""
from __future__ import annotations

import numpy as np

import oracle
from glide_b200 import datasets

INVALID = 0xFFFFFFFF


def small_dataset(kind: str, n: int, dim: int, n_queries: int, seed: int = 7):
    """kind: 'uniform' (continuous, ties improbable) or 'int' (integer valued, ties occur)."""
    if kind == "uniform":
        spec = datasets.DatasetSpec("t", n, dim, n_queries, "uniform", 0, "Euclidean", 32, seed)
    elif kind == "int":
        spec = datasets.DatasetSpec("t", n, dim, n_queries, "int_mixture", 16, "Euclidean", 32, seed)
    elif kind == "scaled":   # the 960-dim config's distribution: N(0,1) centres, sigma 0.3, row scale U[0.5,1.5]
        spec = datasets.DatasetSpec("t", n, dim, n_queries, "scaled_mixture", 12, "Euclidean", 64, seed)
    elif kind == "unit":
        spec = datasets.DatasetSpec("t", n, dim, n_queries, "unit_mixture", 16, "Cosine", 32, seed)
    else:
        raise ValueError(kind)
    return datasets.make(spec)


def exact_partition_knn(reorder_data, seg_start, seg_len, k, metric):
    """Exact kNN inside each partition, partition-local ids, self excluded (int32 like the kNN file)."""
    rows = reorder_data.shape[0]
    knn = np.zeros((rows, k), np.int32)
    for s, l in zip(seg_start, seg_len):
        s, l = int(s), int(l)
        if l == 0:
            continue
        part = reorder_data[s:s + l]
        kk = min(k + 1, l)
        ids = oracle.bruteforce_knn(part, part, kk, metric, want_dists=False)
        for r in range(l):
            row = [int(x) for x in ids[r] if int(x) != r][:k]
            while len(row) < k:  # tiny partitions: pad like nn_descent.cuh:1384-1391 pads invalid ids
                row.append((r + 1 + len(row)) % l)
            knn[s + r] = row
    return knn


def oracle_pipeline(base, centroid_num=4, boundary_factor=1.1, knn_degree=16, graph_degree=16, build_beam=32,
                    refine_beam=64, alpha=1.05, metric=oracle.EUCLIDEAN, order=oracle.ORDER_WARP, seed=3,
                    with_refine=True, route_order=oracle.ORDER_TEAM):
    """partition -> exact kNN per partition -> build -> boundary merge -> reverse -> refine, all on the oracle."""
    n, dim = base.shape
    rng = np.random.default_rng(seed)
    sample = base[rng.permutation(n)[:max(centroid_num * 20, 64)]]
    centroids, _, _ = oracle.kmeans(sample, centroid_num, 10, order=route_order, metric=metric, init=0)
    seg_index, seg_start, seg_len = oracle.define_partition(base, centroids, boundary_factor, metric, route_order)
    reorder_data, mapping = oracle.reorder(base, seg_index, seg_start, int(seg_len[centroid_num]))
    knn = exact_partition_knn(reorder_data, seg_start, seg_len, knn_degree, metric)
    local_sp = np.array([rng.integers(0, max(int(l), 1)) for l in seg_len], np.uint32)
    orig_sp = np.array([mapping[int(seg_start[i]) + int(local_sp[i])] for i in range(centroid_num)], np.uint32)
    p_build = oracle.SearchParams.derive(build_beam, knn_degree)
    graph = oracle.build_rows(reorder_data, knn.view(np.uint32), seg_start, seg_len, local_sp, mapping, n,
                              graph_degree, p_build, alpha, metric, order)
    after_build = graph.copy()
    if seg_len[centroid_num] > 0:
        oracle.build_boundary(reorder_data, knn.view(np.uint32), n, int(local_sp[centroid_num]), mapping, graph,
                              p_build, alpha, metric, order)
    after_boundary = graph.copy()
    oracle.reverse_graph(graph)
    after_reverse = graph.copy()
    p_refine = oracle.SearchParams.derive(refine_beam, knn_degree)  # quirk: hash sized from knn_degree
    if with_refine:
        graph = oracle.refine(base, graph, centroids, orig_sp, p_refine, alpha, metric, order, route_order=route_order)
    return dict(centroids=centroids, seg_index=seg_index, seg_start=seg_start, seg_len=seg_len,
                reorder_data=reorder_data, mapping=mapping, knn=knn, local_sp=local_sp, orig_sp=orig_sp,
                p_build=p_build, p_refine=p_refine, after_build=after_build, after_boundary=after_boundary,
                after_reverse=after_reverse, graph=graph, alpha=alpha, metric=metric, order=order)
