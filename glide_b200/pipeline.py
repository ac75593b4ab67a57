"""The four small-path stages chained in one process: what the reference runs as
``small_preprocess`` -> ``small_knn`` -> ``small_build`` -> ``small_search`` (test.sh:27-33),
with the same parameter derivations as those mains and optional stage files in the
reference's formats and names (small_build.cu:43-48)."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from . import api, io
from .params import IndexParameter, Metric, NNDescentParameter, PartitionParameter, SearchParameter


@dataclass
class BuildConfig:
    """Defaults are the reference's test.sh:10-21."""
    metric: Metric = Metric.Euclidean
    centroid_num: int = 10
    boundary_factor: float = 1.04
    sample_factor: float = 0.01
    knn_degree: int = 32
    graph_degree: int = 32
    relaxant_factor: float = 1.05
    build_beam: int = 64
    refine_beam: int = 128
    nnd_max_iterations: int = 20
    nnd_termination_threshold: float = 0.0001
    nnd_sample: int = 0
    exact_knn_max_rows: int = 0xFFFFFFFF   # partitions up to this size get an exact all-pairs kNN graph
    refine_wave_rows: int = 65536          # refine takes the points in waves of this many consecutive ids (0: one wave)
    seed: int = 0


@dataclass
class BuildResult:
    index: api.GLIDE
    seconds: dict = field(default_factory=dict)   # per stage, kernel time (the reference's convention)
    h_segment_start: np.ndarray | None = None
    h_segment_length: np.ndarray | None = None
    nnd_rounds: int = 0
    d_knn: torch.Tensor | None = None
    d_reorder_data: torch.Tensor | None = None
    d_map: torch.Tensor | None = None

    @property
    def total_seconds(self) -> float:
        return float(sum(self.seconds.values()))


def derive_build_search_params(cfg: BuildConfig) -> tuple[SearchParameter, SearchParameter]:
    """small_build.cu:61-82. Both hash tables are sized from knn_degree, as there."""
    knn = SearchParameter(beam=cfg.build_beam).derive(cfg.knn_degree)
    if cfg.refine_beam:
        refine = SearchParameter(beam=cfg.refine_beam).derive(cfg.knn_degree)
    else:
        refine = SearchParameter(beam=0)
    return knn, refine


def derive_search_params(beam: int, graph_degree: int, top_k: int = 10) -> SearchParameter:
    """small_search.cu:92-107."""
    return SearchParameter(top_k=top_k, beam=beam).derive(graph_degree)


def build_small(ctx: api.Context, d_data: torch.Tensor, cfg: BuildConfig, keep_intermediates: bool = False,
                stage_prefix: str | None = None) -> BuildResult:
    seconds = {}
    pre = api.preprocess(ctx, PartitionParameter(cfg.centroid_num, cfg.boundary_factor, cfg.sample_factor, cfg.metric),
                         d_data, cfg.seed)
    seconds["preprocess"] = pre["seconds"]
    seg_start, seg_len = pre["h_segment_start"], pre["h_segment_length"]
    nnd = NNDescentParameter(cfg.knn_degree, cfg.nnd_max_iterations, cfg.nnd_termination_threshold)
    d_knn, rounds, knn_seconds = api.build_nnd(ctx, nnd, pre["d_reorder_data"], seg_start, seg_len, cfg.metric,
                                               cfg.seed, cfg.nnd_sample, cfg.exact_knn_max_rows)
    seconds["knn"] = knn_seconds
    index = api.GLIDE(ctx, cfg.graph_degree, d_data, pre["d_centroids"], cfg.metric)
    p_knn, p_refine = derive_build_search_params(cfg)
    index.build(IndexParameter(cfg.graph_degree, cfg.knn_degree, cfg.relaxant_factor, cfg.metric), p_knn, p_refine,
                d_knn, seg_start, seg_len, pre["d_map"], pre["d_reorder_data"], cfg.seed, cfg.refine_wave_rows)
    seconds.update(index.stage_seconds)
    if stage_prefix is not None:
        io.save_matrix_data(stage_prefix + ".centroid", pre["d_centroids"].cpu().numpy())
        io.save_segment(stage_prefix + ".segment", seg_start, seg_len)
        io.save_vector_data(stage_prefix + ".map", api.to_u32(pre["d_map"]))
        io.save_matrix_data(stage_prefix + ".reorder", pre["d_reorder_data"].cpu().numpy())
        io.save_matrix_data(stage_prefix + ".knn", d_knn.cpu().numpy())
        io.save_matrix_data(stage_prefix + ".graph", api.to_u32(index.graph_view()))
        io.save_vector_data(stage_prefix + ".sp", api.to_u32(index.start_point_view()))
    res = BuildResult(index, seconds, seg_start, seg_len, rounds)
    if keep_intermediates:
        res.d_knn, res.d_reorder_data, res.d_map = d_knn, pre["d_reorder_data"], pre["d_map"]
    return res


class _GpuBackend:
    """Stage calls of the sharded build on one GPU (see sharded.build_sharded)."""

    def __init__(self, ctx, index, cfg, pre, d_knn, d_local, p_knn, p_refine):
        self.ctx, self.index, self.cfg, self.pre = ctx, index, cfg, pre
        self.knn, self.graph = d_knn, index.d_graph
        self.d_local, self.p_knn, self.p_refine = d_local, p_knn, p_refine
        self.seg_start = np.ascontiguousarray(pre["h_segment_start"], np.uint32)
        self.seg_len = np.ascontiguousarray(pre["h_segment_length"], np.uint32)
        self.nnd_rounds = 0

    def knn_segments(self, lo, hi):
        import ctypes as C
        ctx, cfg = self.ctx, self.cfg
        first = int(self.seg_start[lo])
        rows = int(self.seg_start[hi - 1]) + int(self.seg_len[hi - 1]) - first
        if rows == 0:
            return 0.0
        start = np.ascontiguousarray(self.seg_start[lo:hi] - np.uint32(first))
        length = np.ascontiguousarray(self.seg_len[lo:hi])
        d_rows = self.pre["d_reorder_data"][first:first + rows]
        out = self.knn[first:first + rows]
        rounds = C.c_uint32(0)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_build_nnd_range(
            ctx.handle, d_rows.data_ptr(), rows, d_rows.shape[1], start.ctypes.data, length.ctypes.data, hi - lo,
            self.knn.shape[1], cfg.nnd_max_iterations, cfg.nnd_termination_threshold, cfg.nnd_sample,
            cfg.exact_knn_max_rows, cfg.seed, int(cfg.metric), first, out.data_ptr(), C.byref(rounds)))
        self.nnd_rounds = int(rounds.value)
        return ctx.last_kernel_seconds

    def build_rows(self, first_row, row_count, out):
        import ctypes as C
        ctx, idx, pre = self.ctx, self.index, self.pre
        if row_count == 0:
            return 0.0
        pc = api._params_c(self.p_knn)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_subgraph_build_rows(
            ctx.handle, pre["d_reorder_data"].data_ptr(), pre["d_reorder_data"].shape[0], idx.dim(), self.knn.data_ptr(),
            self.knn.shape[1], self.seg_start.ctypes.data, self.seg_len.ctypes.data, self.seg_start.size,
            self.d_local.data_ptr(), pre["d_map"].data_ptr(), idx.num(), idx.graph_degree(), C.byref(pc),
            self.cfg.relaxant_factor, int(self.cfg.metric), first_row, row_count, out.data_ptr()))
        return ctx.last_kernel_seconds

    def build_boundary(self, first_row, row_count):
        import ctypes as C
        ctx, idx, pre = self.ctx, self.index, self.pre
        if row_count == 0:
            return 0.0
        pc = api._params_c(self.p_knn)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_subgraph_build_range(
            ctx.handle, pre["d_reorder_data"].data_ptr(), pre["d_reorder_data"].shape[0], idx.dim(), self.knn.data_ptr(),
            self.knn.shape[1], self.seg_start.ctypes.data, self.seg_len.ctypes.data, self.seg_start.size,
            self.d_local.data_ptr(), pre["d_map"].data_ptr(), idx.num(), idx.graph_degree(), C.byref(pc),
            self.cfg.relaxant_factor, int(self.cfg.metric), first_row, row_count, idx.d_graph.data_ptr()))
        return ctx.last_kernel_seconds

    def reverse(self):
        return api.reverse_graph(self.ctx, self.index.d_graph)

    def refine_rows(self, first, count, out):
        import ctypes as C
        ctx, idx = self.ctx, self.index
        if count == 0:
            return 0.0
        pc = api._params_c(self.p_refine)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_refine_rows(ctx.handle, idx.d_data.data_ptr(), idx.num(), idx.dim(), idx.d_graph.data_ptr(),
                                            idx.graph_degree(), idx.d_centroids.data_ptr(), idx.centroid_num(),
                                            idx.d_start_points.data_ptr(), C.byref(pc), self.cfg.relaxant_factor,
                                            int(self.cfg.metric), first, count, out.data_ptr()))
        return ctx.last_kernel_seconds


def build_small_sharded(ctx: api.Context, d_data: torch.Tensor, cfg: BuildConfig, coll=None) -> BuildResult:
    """build_small with the kNN stage, the subgraph build and refinement split over the ranks of
    `coll` (sharded.GlideCollectives over the context's communicator; None: one rank); every rank
    ends with the full index, equal to the single-GPU one bit for bit."""
    from . import sharded
    if coll is None:
        coll = sharded.Collectives()
    seconds = {}
    pre = api.preprocess(ctx, PartitionParameter(cfg.centroid_num, cfg.boundary_factor, cfg.sample_factor, cfg.metric),
                         d_data, cfg.seed)
    seconds["preprocess"] = pre["seconds"]
    seg_start, seg_len = pre["h_segment_start"], pre["h_segment_length"]
    rows = pre["d_reorder_data"].shape[0]
    degree = min(cfg.knn_degree, NNDescentParameter(cfg.knn_degree).intermediate_graph_degree)
    d_knn = torch.zeros((rows, degree), dtype=torch.int32, device=ctx.torch_device)
    index = api.GLIDE(ctx, cfg.graph_degree, d_data, pre["d_centroids"], cfg.metric)
    index.d_graph.fill_(-1)
    p_knn, p_refine = derive_build_search_params(cfg)
    h_map = api.to_u32(pre["d_map"])
    local, original = api.start_point_select(seg_start, seg_len, h_map, cfg.seed)
    index.d_start_points = api.from_u32(ctx, original)
    backend = _GpuBackend(ctx, index, cfg, pre, d_knn, api.from_u32(ctx, local), p_knn, p_refine)
    num = index.num()
    map_ids = torch.from_numpy(h_map.astype(np.int64)).to(ctx.torch_device)
    torch.cuda.synchronize(ctx.torch_device)
    exact_max = 16384 if cfg.exact_knn_max_rows == 0xFFFFFFFF else cfg.exact_knn_max_rows
    seconds.update(sharded.build_sharded(backend, coll, num, int(seg_len[-1]), seg_start, seg_len, map_ids,
                                         do_refine=cfg.refine_beam != 0, wave_rows=cfg.refine_wave_rows,
                                         exact_max_rows=exact_max))
    torch.cuda.synchronize(ctx.torch_device)
    index.stage_seconds = {k: v for k, v in seconds.items() if k not in ("preprocess", "knn")}
    return BuildResult(index, seconds, seg_start, seg_len, backend.nnd_rounds)
