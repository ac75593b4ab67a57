"""Large path: the data set lives in host memory and partitions are streamed through the GPU
one at a time (reference ``GLIDE_large``, glide_large.cuh:14-212, glide_large_impl.cuh:14-507;
``preprocess_for_large`` partition.cuh:417-447; ``build_knn_for_large`` nn_descent.cuh:1515-1581).

Differences from the reference a caller will notice: data are fp32 (the reference's large
path is uint8), every random choice is seeded, and no trailing rows are dropped (the reference
processes floor(N / batch_num) * batch_num rows, partition.cuh:231).
Partitions are disjoint (no boundary copies) and every subgraph uses partition-local ids; a
query visits every partition whose centroid distance is within ``boundary_factor`` of the
nearest one (at least ``min_segment_num`` partitions) and the per-partition results are folded
into one running top-k.
"""
from __future__ import annotations

import numpy as np
import torch

from . import api
from .params import IndexParameter, Metric, NNDescentParameter, SearchParameter


def _splitmix(seed: int):
    mask = (1 << 64) - 1
    state = seed & mask
    while True:
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        yield z ^ (z >> 31)


def preprocess_for_large(ctx: api.Context, h_data: np.ndarray, centroid_num: int, sample_factor: float,
                         batch_num: int = 10, metric: Metric = Metric.Euclidean, seed: int = 0):
    """Centroids from a host-gathered sample, nearest-centroid assignment batch by batch on the GPU
    (no boundary test, partition_kernel.cuh:122-162), then the rows grouped by partition in ascending
    row order. Returns dict(h_reorder_data, h_map, h_segment_start, h_segment_length, h_centroids, seconds)."""
    n, dim = h_data.shape
    sample_num = max(centroid_num, int(n * sample_factor))
    ids = api.sample_ids(n, sample_num, seed)
    d_sample = torch.from_numpy(np.ascontiguousarray(h_data[ids])).to(ctx.torch_device)
    d_centroids, _, _ = api.kmeans_fit(ctx, d_sample, centroid_num, 0, metric, 1)
    seconds = ctx.last_kernel_seconds
    nearest = np.empty(n, np.uint32)
    batch = (n + batch_num - 1) // batch_num
    for lo in range(0, n, batch):
        hi = min(n, lo + batch)
        d_rows = torch.from_numpy(np.ascontiguousarray(h_data[lo:hi])).to(ctx.torch_device)
        d_seg, _, _ = api.define_partition(ctx, d_rows, d_centroids, -1.0, metric)
        seconds += ctx.last_kernel_seconds
        nearest[lo:hi] = api.to_u32(d_seg)[:, 0]
    order = np.argsort(nearest, kind="stable").astype(np.uint32)   # ascending row id inside a partition
    seg_len = np.bincount(nearest, minlength=centroid_num).astype(np.uint32)
    seg_start = np.zeros(centroid_num, np.uint32)
    seg_start[1:] = np.cumsum(seg_len[:-1], dtype=np.uint64).astype(np.uint32)
    return dict(h_reorder_data=np.ascontiguousarray(h_data[order]), h_map=order, h_segment_start=seg_start,
                h_segment_length=seg_len, h_centroids=d_centroids.cpu().numpy(), seconds=seconds)


def build_knn_for_large(ctx: api.Context, param: NNDescentParameter, h_reorder_data: np.ndarray, h_segment_start,
                        h_segment_length, metric: Metric = Metric.Euclidean, seed: int = 0,
                        exact_max_rows: int = 0xFFFFFFFF):
    """kNN graph of every partition, one resident partition at a time. Returns (h_knn int32, seconds)."""
    rows = h_reorder_data.shape[0]
    degree = min(param.graph_degree, param.intermediate_graph_degree)
    h_knn = np.zeros((rows, degree), np.int32)
    seconds = 0.0
    for s, l in zip(h_segment_start, h_segment_length):
        s, l = int(s), int(l)
        if l == 0:
            continue
        d_part = torch.from_numpy(h_reorder_data[s:s + l]).to(ctx.torch_device)
        d_knn, _, sec = api.build_nnd(ctx, param, d_part, np.array([0], np.uint32), np.array([l], np.uint32), metric,
                                      seed, 0, exact_max_rows)
        seconds += sec
        h_knn[s:s + l] = d_knn.cpu().numpy()
    return h_knn, seconds


class GLIDE_large:
    """Host-resident index over disjoint partitions (glide_large.cuh:14-212)."""

    def __init__(self, ctx: api.Context, graph_degree: int, metric: Metric, h_reorder_data: np.ndarray, h_map,
                 h_centroids, h_segment_start, h_segment_length):
        self.ctx, self.metric = ctx, metric
        self.h_data = np.ascontiguousarray(h_reorder_data, np.float32)
        self.h_map = np.ascontiguousarray(h_map, np.uint32)
        self.h_centroids = np.ascontiguousarray(h_centroids, np.float32)
        self.seg_start = np.ascontiguousarray(h_segment_start, np.uint32)
        self.seg_len = np.ascontiguousarray(h_segment_length, np.uint32)
        self.h_graph = np.full((self.h_data.shape[0], graph_degree), api.INVALID, np.uint32)
        self.h_start_points = np.zeros(self.seg_start.size, np.uint32)
        self.stage_seconds: dict[str, float] = {}

    def num(self): return self.h_data.shape[0]
    def dim(self): return self.h_data.shape[1]
    def graph_degree(self): return self.h_graph.shape[1]
    def segment_num(self): return self.seg_start.size
    def centroids_num(self): return self.h_centroids.shape[0]
    def graph_view(self): return self.h_graph
    def start_point_view(self): return self.h_start_points

    def load(self, h_graph, h_start_points):
        self.h_graph = np.ascontiguousarray(h_graph, np.uint32)
        self.h_start_points = np.ascontiguousarray(h_start_points, np.uint32)

    def start_point_select(self, seed: int):
        """One seeded random member per partition, as a partition-local id (glide_large_impl.cuh:50-77)."""
        gen = _splitmix(seed)
        for i, l in enumerate(self.seg_len):
            r = next(gen)
            self.h_start_points[i] = r % int(l) if l else 0

    def build(self, build_param: IndexParameter, search_param_knn: SearchParameter,
              search_param_refine: SearchParameter, h_knn_graph: np.ndarray, seed: int = 0):
        """Per resident partition: H2D rows and kNN rows, build_for_large_kernel, reverse edges,
        refine_for_large_kernel, D2H rows (glide_large_impl.cuh:79-328). Returns kernel seconds."""
        ctx = self.ctx
        self.start_point_select(seed)
        t = dict(subgraph_build=0.0, reverse_graph=0.0, refine=0.0)
        for i, (s, l) in enumerate(zip(self.seg_start, self.seg_len)):
            s, l = int(s), int(l)
            if l == 0:
                continue
            d_part = torch.from_numpy(self.h_data[s:s + l]).to(ctx.torch_device)
            d_knn = api.from_u32(ctx, np.ascontiguousarray(h_knn_graph[s:s + l]).view(np.uint32))
            sp = int(self.h_start_points[i])
            d_graph = api.build_partition(ctx, d_part, d_knn, sp, self.graph_degree(), search_param_knn,
                                          build_param.relaxant_factor, self.metric)
            t["subgraph_build"] += ctx.last_kernel_seconds
            t["reverse_graph"] += api.reverse_graph(ctx, d_graph)
            if search_param_refine.beam != 0:
                t["refine"] += api.refine_partition(ctx, d_part, d_graph, sp, search_param_refine,
                                                    build_param.relaxant_factor, self.metric)
            self.h_graph[s:s + l] = api.to_u32(d_graph)
        self.stage_seconds = t
        return sum(t.values())

    def search(self, param: SearchParameter, min_segment_num: int, boundary_factor: float, d_query: torch.Tensor):
        """glide_large_impl.cuh:355-507. Returns (ids uint32 [Q,k] original ids, dists [Q,k], kernel seconds)."""
        ctx = self.ctx
        q = d_query.shape[0]
        d_centroids = torch.from_numpy(self.h_centroids).to(ctx.torch_device)
        d_routes = api.select_segments(ctx, d_query, d_centroids, min_segment_num, boundary_factor, self.metric)
        seconds = ctx.last_kernel_seconds
        d_final_ids = api._u32_tensor(ctx, (q, param.top_k))
        d_final_ids.fill_(-1)
        d_final_d = torch.full((q, param.top_k), torch.finfo(torch.float32).max, device=ctx.torch_device)
        for i, (s, l) in enumerate(zip(self.seg_start, self.seg_len)):
            s, l = int(s), int(l)
            if l == 0:
                continue
            d_part = torch.from_numpy(self.h_data[s:s + l]).to(ctx.torch_device)
            d_graph = api.from_u32(ctx, self.h_graph[s:s + l])
            d_map = api.from_u32(ctx, self.h_map[s:s + l])
            seconds += api.search_on_sub(ctx, d_part, d_graph, d_map, int(self.h_start_points[i]), d_query, d_routes, i,
                                         param, d_final_ids, d_final_d, self.metric)
        return api.to_u32(d_final_ids), d_final_d.cpu().numpy(), seconds
