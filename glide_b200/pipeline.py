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
                d_knn, seg_start, seg_len, pre["d_map"], pre["d_reorder_data"], cfg.seed)
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
        self.ctx, self.index, self.cfg, self.pre, self.d_knn = ctx, index, cfg, pre, d_knn
        self.d_local, self.p_knn, self.p_refine = d_local, p_knn, p_refine

    def build_range(self, first_row, row_count):
        import ctypes as C
        ctx, idx, pre = self.ctx, self.index, self.pre
        if row_count == 0:
            return 0.0
        seg_start = np.ascontiguousarray(pre["h_segment_start"], np.uint32)
        seg_len = np.ascontiguousarray(pre["h_segment_length"], np.uint32)
        pc = api._params_c(self.p_knn)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_subgraph_build_range(
            ctx.handle, pre["d_reorder_data"].data_ptr(), pre["d_reorder_data"].shape[0], idx.dim(), self.d_knn.data_ptr(),
            self.d_knn.shape[1], seg_start.ctypes.data, seg_len.ctypes.data, seg_start.size, self.d_local.data_ptr(),
            pre["d_map"].data_ptr(), idx.num(), idx.graph_degree(), C.byref(pc), self.cfg.relaxant_factor,
            int(self.cfg.metric), first_row, row_count, idx.d_graph.data_ptr()))
        return ctx.last_kernel_seconds

    def reverse(self):
        return api.reverse_graph(self.ctx, self.index.d_graph)

    def refine_range(self, snapshot, first, count):
        import ctypes as C
        ctx, idx = self.ctx, self.index
        pc = api._params_c(self.p_refine)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_refine_range(ctx.handle, idx.d_data.data_ptr(), idx.num(), idx.dim(), snapshot.data_ptr(),
                                             idx.d_graph.data_ptr(), idx.graph_degree(), idx.d_centroids.data_ptr(),
                                             idx.centroid_num(), idx.d_start_points.data_ptr(), C.byref(pc),
                                             self.cfg.relaxant_factor, int(self.cfg.metric), first, count))
        return ctx.last_kernel_seconds


def build_small_sharded(ctx: api.Context, d_data: torch.Tensor, cfg: BuildConfig, dist=None, world: int = 1,
                        rank: int = 0) -> BuildResult:
    """build_small with the subgraph build and refinement split over `world` ranks (one GPU each)
    and their rows exchanged over torch.distributed; every rank ends with the full index, equal to
    the single-GPU one."""
    from . import sharded
    seconds = {}
    pre = api.preprocess(ctx, PartitionParameter(cfg.centroid_num, cfg.boundary_factor, cfg.sample_factor, cfg.metric),
                         d_data, cfg.seed)
    seconds["preprocess"] = pre["seconds"]
    seg_start, seg_len = pre["h_segment_start"], pre["h_segment_length"]
    nnd = NNDescentParameter(cfg.knn_degree, cfg.nnd_max_iterations, cfg.nnd_termination_threshold)
    d_knn, rounds, seconds["knn"] = api.build_nnd(ctx, nnd, pre["d_reorder_data"], seg_start, seg_len, cfg.metric,
                                                  cfg.seed, cfg.nnd_sample, cfg.exact_knn_max_rows)
    index = api.GLIDE(ctx, cfg.graph_degree, d_data, pre["d_centroids"], cfg.metric)
    p_knn, p_refine = derive_build_search_params(cfg)
    h_map = api.to_u32(pre["d_map"])
    local, original = api.start_point_select(seg_start, seg_len, h_map, cfg.seed)
    index.d_start_points = api.from_u32(ctx, original)
    backend = _GpuBackend(ctx, index, cfg, pre, d_knn, api.from_u32(ctx, local), p_knn, p_refine)
    coll = sharded.Collectives(dist, world, rank)
    num = index.num()
    map_ids = torch.from_numpy(h_map.astype(np.int64)).to(ctx.torch_device)
    torch.cuda.synchronize(ctx.torch_device)
    seconds.update(sharded.build_sharded(backend, coll, num, int(seg_len[-1]), index.d_graph, map_ids,
                                         do_refine=cfg.refine_beam != 0))
    torch.cuda.synchronize(ctx.torch_device)
    index.stage_seconds = {k: v for k, v in seconds.items() if k not in ("preprocess", "knn")}
    return BuildResult(index, seconds, seg_start, seg_len, rounds)
