"""Host-side mirror of the reference's C++ API for the hot path, over the C ABI.

Names and argument meaning follow the reference: ``preprocess`` (partition.cuh:159-193),
``build_nnd`` (nn_descent.cuh:1405-1467), class ``GLIDE`` with ``load`` / ``build`` /
``search`` and accessors (glide.cuh:14-189, glide_impl.cuh:15-454). Device matrices are
torch CUDA tensors (torch is used for device memory only); host vectors are numpy.
Differences a caller will notice: every random choice takes a seed (the reference seeds
from ``std::random_device``), the device is a parameter, and stage times are returned
instead of being appended to a result file by the library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from .params import IndexParameter, Metric, NNDescentParameter, PartitionParameter, SearchParameter

INVALID = 0xFFFFFFFF


class GlideError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"glide_b200 error {code}: {message}")
        self.code = code


class UnsupportedError(GlideError, ValueError):
    """Unsupported beam / graph_degree / centroid count: the reference throws
    std::invalid_argument here (kernel_config.cuh:47-48, :59-60, :232-233)."""


def _ptr(t) -> int:
    if t is None:
        return 0
    # every buffer of the C ABI holds 4-byte elements (fp32, u32, i32): anything else would be read as garbage
    if isinstance(t, torch.Tensor):
        if not t.is_contiguous() or t.element_size() != 4:
            raise TypeError(f"tensor must be contiguous with 4-byte elements, got {t.dtype}, contiguous={t.is_contiguous()}")
        return t.data_ptr()
    if isinstance(t, np.ndarray):
        if not t.flags.c_contiguous or t.dtype.itemsize != 4:
            raise TypeError(f"array must be C-contiguous with 4-byte elements, got {t.dtype}")
        return t.ctypes.data
    raise TypeError(type(t))


def _params_c(p: SearchParameter) -> _lib.SearchParamsC:
    return _lib.SearchParamsC(p.top_k, p.beam, p.max_iterations, p.min_iterations, p.hash_bit, p.hash_reset_interval)


class Context:
    """One device, one stream, one scratch arena (``glide_ctx``)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("glide_b200 needs a CUDA device; there is no CPU fallback")
        self.device = device
        self.torch_device = torch.device("cuda", device)
        torch.cuda.set_device(device)
        torch.zeros(1, device=self.torch_device)  # make sure the primary context exists
        h = C.c_void_p()
        rc = self.lib.glide_ctx_create(device, C.byref(h))
        if rc != 0:
            raise GlideError(rc, "glide_ctx_create failed")
        self.handle = h

    def close(self):
        if getattr(self, "handle", None):
            self.lib.glide_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc: int):
        if rc != 0:
            msg = self.lib.glide_last_error(self.handle).decode()
            raise (UnsupportedError if rc == -2 else GlideError)(rc, msg)

    def sync_inputs(self):
        """Inputs are produced on torch's stream; the library runs on its own."""
        torch.cuda.current_stream(self.torch_device).synchronize()

    @property
    def last_kernel_seconds(self) -> float:
        return float(self.lib.glide_last_kernel_ms(self.handle)) / 1000.0

    @property
    def tc_knn_fallbacks(self) -> int:
        """kNN stages the tensor-core kernel handed back to the fp32 kernels (0 in normal operation)."""
        return int(self.lib.glide_tc_knn_fallbacks(self.handle))

    def empty(self, shape, dtype) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype, device=self.torch_device)

    def init_comm(self, dist=None, world: int = 1, rank: int = 0):
        """Give the context an NCCL communicator over `world` ranks (one process per GPU). The 128-byte
        rendezvous token is made by rank 0 and carried to the others through torch.distributed's
        process group `dist` (any backend); from then on torch.distributed plays no part in the data
        path. One small collective is run so that NCCL's lazy set-up is paid here."""
        token = np.zeros(128, np.uint8)
        if rank == 0:
            rc = self.lib.glide_comm_unique_id(token.ctypes.data)
            if rc != 0:
                raise GlideError(rc, "glide_comm_unique_id failed (libnccl.so.2 not found?)")
        if world > 1:
            box = [token.tobytes()]
            dist.broadcast_object_list(box, src=0)
            token = np.frombuffer(box[0], np.uint8).copy()
        self.check(self.lib.glide_comm_init(self.handle, token.ctypes.data, world, rank))
        warm = torch.zeros(2, dtype=torch.int64, device=self.torch_device)
        self.sync_inputs()
        self.check(self.lib.glide_comm_all_reduce_u64(self.handle, warm.data_ptr(), 2, 0))
        self.check(self.lib.glide_ctx_synchronize(self.handle))

    def all_reduce_u64(self, t: torch.Tensor, op: str = "sum"):
        """In place over the ranks of the context's communicator; t: int64/uint64 tensor on the device."""
        assert t.element_size() == 8 and t.is_contiguous()
        self.sync_inputs()
        self.check(self.lib.glide_comm_all_reduce_u64(self.handle, t.data_ptr(), t.numel(), {"sum": 0, "max": 1, "min": 2}[op]))
        self.check(self.lib.glide_ctx_synchronize(self.handle))
        return t

    def enable_counters(self, on: bool):
        self.lib.glide_enable_counters(self.handle, 1 if on else 0)

    def read_counters(self) -> tuple[int, int, int, int]:
        """(rows read while searching, expansions, rows read while pruning, points whose beam
        ended unfilled) of the last search / build / refine call."""
        out = (C.c_uint64 * 4)()
        self.check(self.lib.glide_read_counters(self.handle, out))
        return int(out[0]), int(out[1]), int(out[2]), int(out[3])


# torch has no uint32 arithmetic, but plain storage works; ids live in int32 tensors
# viewed as uint32 bit patterns.
def _u32_tensor(ctx: Context, shape) -> torch.Tensor:
    return ctx.empty(shape, torch.int32)


def to_u32(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy().view(np.uint32)


def from_u32(ctx: Context, a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32)).to(ctx.torch_device)


def sample_ids(n: int, sample_num: int, seed: int) -> np.ndarray:
    out = np.empty(sample_num, np.uint32)
    rc = _lib.load().glide_sample_ids(n, sample_num, seed, _ptr(out))
    if rc != 0:
        raise GlideError(rc, "glide_sample_ids: bad argument")
    return out


def get_centroids(ctx: Context, d_data: torch.Tensor, centroid_num: int, sample_factor: float, seed: int = 0,
                  max_iter: int = 0, metric: Metric = Metric.Euclidean):
    """partition.cuh:8-59. Returns (d_centroids, rounds)."""
    n, dim = d_data.shape
    d_centroids = ctx.empty((centroid_num, dim), torch.float32)
    rounds = C.c_uint32(0)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_get_centroids(ctx.handle, _ptr(d_data), n, dim, centroid_num, sample_factor, seed, max_iter,
                                          int(metric), _ptr(d_centroids), C.byref(rounds)))
    return d_centroids, rounds.value


def kmeans_fit(ctx: Context, d_sample: torch.Tensor, centroid_num: int, max_iter: int = 0,
               metric: Metric = Metric.Euclidean, init: int = 1):
    n, dim = d_sample.shape
    d_centroids = ctx.empty((centroid_num, dim), torch.float32)
    d_labels = _u32_tensor(ctx, (n,))
    rounds = C.c_uint32(0)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_kmeans_fit(ctx.handle, _ptr(d_sample), n, dim, centroid_num, max_iter, int(metric), init,
                                       _ptr(d_centroids), _ptr(d_labels), C.byref(rounds)))
    return d_centroids, d_labels, rounds.value


def define_partition(ctx: Context, d_data: torch.Tensor, d_centroids: torch.Tensor, boundary_factor: float,
                     metric: Metric = Metric.Euclidean):
    """partition.cuh:61-116. Returns (d_segment_index [n,3], h_segment_start, h_segment_length), C+1 entries."""
    n, dim = d_data.shape
    c = d_centroids.shape[0]
    d_seg_index = _u32_tensor(ctx, (n, 3))
    seg_start = np.zeros(c + 1, np.uint32)
    seg_len = np.zeros(c + 1, np.uint32)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_define_partition(ctx.handle, _ptr(d_data), n, dim, _ptr(d_centroids), c, boundary_factor,
                                             int(metric), _ptr(d_seg_index), _ptr(seg_start), _ptr(seg_len)))
    return d_seg_index, seg_start, seg_len


def reorder(ctx: Context, d_data: torch.Tensor, d_seg_index: torch.Tensor, seg_start: np.ndarray, boundary_num: int):
    """partition.cuh:118-157. Returns (d_reorder_data, d_map)."""
    n, dim = d_data.shape
    c = seg_start.size - 1
    d_reorder = ctx.empty((n + boundary_num, dim), torch.float32)
    d_map = _u32_tensor(ctx, (n + boundary_num,))
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_reorder(ctx.handle, _ptr(d_data), n, dim, _ptr(d_seg_index), _ptr(seg_start), c,
                                    _ptr(d_reorder), _ptr(d_map)))
    return d_reorder, d_map


def preprocess(ctx: Context, param: PartitionParameter, d_data: torch.Tensor, seed: int = 0):
    """``preprocess`` of partition.cuh:159-193: centroids, assignment with boundary test, reorder.

    Returns a dict with d_reorder_data, d_map, h_segment_start, h_segment_length (C+1
    entries, the last is the boundary segment), d_centroids and the kernel seconds.
    """
    seconds = 0.0
    d_centroids, _ = get_centroids(ctx, d_data, param.centroid_num, param.sample_factor, seed, 0, param.metric)
    seconds += ctx.last_kernel_seconds
    d_seg_index, seg_start, seg_len = define_partition(ctx, d_data, d_centroids, param.boundary_factor, param.metric)
    seconds += ctx.last_kernel_seconds
    d_reorder, d_map = reorder(ctx, d_data, d_seg_index, seg_start, int(seg_len[param.centroid_num]))
    seconds += ctx.last_kernel_seconds
    return dict(d_reorder_data=d_reorder, d_map=d_map, h_segment_start=seg_start, h_segment_length=seg_len,
                d_centroids=d_centroids, seconds=seconds)


def build_nnd(ctx: Context, param: NNDescentParameter, d_data: torch.Tensor, h_segment_start: np.ndarray,
              h_segment_length: np.ndarray, metric: Metric = Metric.Euclidean, seed: int = 0, sample: int = 0,
              exact_max_rows: int = 0xFFFFFFFF):
    """``build_nnd`` of nn_descent.cuh:1405-1467. Returns (d_knn int32 [rows, degree], rounds, seconds).

    As in the reference the output degree is min(graph_degree, intermediate_graph_degree)
    (nn_descent.cuh:1423-1425) and ids are partition-local. Partitions of at most
    ``exact_max_rows`` rows are solved exactly by all pairs (default 16384; 0 = descent everywhere).
    """
    rows, dim = d_data.shape
    degree = min(param.graph_degree, param.intermediate_graph_degree)
    d_knn = ctx.empty((rows, degree), torch.int32)
    rounds = C.c_uint32(0)
    seg_start = np.ascontiguousarray(h_segment_start, np.uint32)
    seg_len = np.ascontiguousarray(h_segment_length, np.uint32)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_build_nnd(ctx.handle, _ptr(d_data), rows, dim, _ptr(seg_start), _ptr(seg_len), seg_start.size,
                                      degree, param.max_iterations, param.termination_threshold, sample,
                                      exact_max_rows, seed, int(metric), _ptr(d_knn), C.byref(rounds)))
    return d_knn, rounds.value, ctx.last_kernel_seconds


def bruteforce_knn(ctx: Context, d_base: torch.Tensor, d_queries: torch.Tensor, k: int,
                   metric: Metric = Metric.Euclidean):
    """Exact kNN (ground truth). Returns (ids uint32-as-int32 [Q,k], dists [Q,k])."""
    n, dim = d_base.shape
    q = d_queries.shape[0]
    ids = _u32_tensor(ctx, (q, k))
    dists = ctx.empty((q, k), torch.float32)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_bruteforce_knn(ctx.handle, _ptr(d_base), n, _ptr(d_queries), q, dim, k, int(metric),
                                           _ptr(ids), _ptr(dists)))
    return ids, dists


def start_point_select(h_segment_start, h_segment_length, h_map, seed: int):
    """glide_impl.cuh:43-73. Returns (local ids per segment [S], original ids per centroid [S-1])."""
    seg_start = np.ascontiguousarray(h_segment_start, np.uint32)
    seg_len = np.ascontiguousarray(h_segment_length, np.uint32)
    h_map = np.ascontiguousarray(h_map, np.uint32)
    s = seg_start.size
    local = np.zeros(s, np.uint32)
    original = np.zeros(max(s - 1, 1), np.uint32)
    rc = _lib.load().glide_start_point_select(_ptr(seg_start), _ptr(seg_len), s, _ptr(h_map), seed, _ptr(local),
                                              _ptr(original))
    if rc != 0:
        raise GlideError(rc, "glide_start_point_select: bad argument")
    return local, original[:s - 1]


def subgraph_build_and_merge(ctx: Context, d_reorder_data, d_knn, h_segment_start, h_segment_length,
                             d_start_points_local, d_map, num: int, d_graph, p: SearchParameter,
                             relaxant_factor: float, metric: Metric = Metric.Euclidean, skip_boundary: bool = False):
    """glide_impl.cuh:75-192 on caller-owned buffers; d_graph (num x degree) must be all 0xffffffff."""
    seg_start = np.ascontiguousarray(h_segment_start, np.uint32)
    seg_len = np.ascontiguousarray(h_segment_length, np.uint32)
    pc = _params_c(p)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_subgraph_build_and_merge(
        ctx.handle, _ptr(d_reorder_data), d_reorder_data.shape[0], d_reorder_data.shape[1], _ptr(d_knn),
        d_knn.shape[1], _ptr(seg_start), _ptr(seg_len), seg_start.size, _ptr(d_start_points_local), _ptr(d_map), num,
        d_graph.shape[1], C.byref(pc), relaxant_factor, int(metric), 1 if skip_boundary else 0, _ptr(d_graph)))
    return ctx.last_kernel_seconds


def reverse_graph(ctx: Context, d_graph):
    """glide_impl.cuh:194-256, in place."""
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_reverse_graph(ctx.handle, _ptr(d_graph), d_graph.shape[0], d_graph.shape[1]))
    return ctx.last_kernel_seconds


def refine(ctx: Context, d_data, d_graph, d_centroids, d_start_points, p: SearchParameter, relaxant_factor: float,
           metric: Metric = Metric.Euclidean, wave_rows: int | None = None):
    """glide_impl.cuh:258-317, in place. wave_rows: points are refined in waves of that many consecutive
    ids, each wave reading the rows the earlier ones wrote (None: the library's default of 65,536;
    0: one wave)."""
    pc = _params_c(p)
    ctx.sync_inputs()
    args = (ctx.handle, _ptr(d_data), d_data.shape[0], d_data.shape[1], _ptr(d_graph), d_graph.shape[1], _ptr(d_centroids),
            d_centroids.shape[0], _ptr(d_start_points), C.byref(pc), relaxant_factor, int(metric))
    if wave_rows is None:
        ctx.check(ctx.lib.glide_refine(*args))
    else:
        ctx.check(ctx.lib.glide_refine_waves(*args, wave_rows))
    return ctx.last_kernel_seconds


def search(ctx: Context, d_data, d_graph, d_centroids, d_start_points, d_queries, p: SearchParameter,
           metric: Metric = Metric.Euclidean):
    """glide_impl.cuh:370-454 on caller-owned device buffers. Returns (d_ids, d_dists, seconds)."""
    q = d_queries.shape[0]
    d_ids = _u32_tensor(ctx, (q, p.top_k))
    d_dists = ctx.empty((q, p.top_k), torch.float32)
    pc = _params_c(p)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_search(ctx.handle, _ptr(d_data), d_data.shape[0], d_data.shape[1], _ptr(d_graph),
                                   d_graph.shape[1], _ptr(d_centroids), d_centroids.shape[0], _ptr(d_start_points),
                                   _ptr(d_queries), q, C.byref(pc), int(metric), _ptr(d_ids), _ptr(d_dists)))
    return d_ids, d_dists, ctx.last_kernel_seconds


def select_segments(ctx: Context, d_queries, d_centroids, min_segment_num: int, boundary_factor: float,
                    metric: Metric = Metric.Euclidean):
    """search_kernel.cuh:546-607. Returns d_segment_ids [Q, C]."""
    q, dim = d_queries.shape
    c = d_centroids.shape[0]
    out = _u32_tensor(ctx, (q, c))
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_select_segments(ctx.handle, _ptr(d_queries), q, dim, _ptr(d_centroids), c, min_segment_num,
                                            boundary_factor, int(metric), _ptr(out)))
    return out


def search_on_sub(ctx: Context, d_data, d_graph, d_map, start_point: int, d_queries, d_segment_ids, segment_id: int,
                  p: SearchParameter, d_final_ids, d_final_dists, metric: Metric = Metric.Euclidean):
    """search_kernel.cuh:653-765: one resident partition, folds into the running top-k."""
    pc = _params_c(p)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_search_on_sub(ctx.handle, _ptr(d_data), d_data.shape[1], _ptr(d_graph), d_graph.shape[1],
                                          _ptr(d_map), start_point, _ptr(d_queries), d_queries.shape[0],
                                          _ptr(d_segment_ids), d_segment_ids.shape[1], segment_id, C.byref(pc),
                                          int(metric), _ptr(d_final_ids), _ptr(d_final_dists)))
    return ctx.last_kernel_seconds


def build_partition(ctx: Context, d_data, d_knn, start_point: int, graph_degree: int, p: SearchParameter,
                    relaxant_factor: float, metric: Metric = Metric.Euclidean):
    """build_for_large_kernel, graph_kernel.cuh:675-728. Returns d_graph [num, graph_degree], local ids."""
    num, dim = d_data.shape
    d_graph = _u32_tensor(ctx, (num, graph_degree))
    d_graph.fill_(-1)
    pc = _params_c(p)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_build_partition(ctx.handle, _ptr(d_data), num, dim, _ptr(d_knn), d_knn.shape[1], start_point,
                                            graph_degree, C.byref(pc), relaxant_factor, int(metric), _ptr(d_graph)))
    return d_graph


def refine_partition(ctx: Context, d_data, d_graph, start_point: int, p: SearchParameter, relaxant_factor: float,
                     metric: Metric = Metric.Euclidean):
    """refine_for_large_kernel, graph_kernel.cuh:730-821, in place."""
    pc = _params_c(p)
    ctx.sync_inputs()
    ctx.check(ctx.lib.glide_refine_partition(ctx.handle, _ptr(d_data), d_data.shape[0], d_data.shape[1], _ptr(d_graph),
                                             d_graph.shape[1], start_point, C.byref(pc), relaxant_factor, int(metric)))
    return ctx.last_kernel_seconds


def calculate_recall(neighbors: np.ndarray, truth: np.ndarray, top_k: int) -> float:
    """small_search.cu:14-36: mean over queries of |result[:k] ∩ truth[:k]| / k."""
    nb = np.asarray(neighbors)[:, :top_k]
    tr = np.asarray(truth)[:, :top_k]
    hits = (nb[:, :, None] == tr[:, None, :]).any(axis=2).sum(axis=1)
    return float(np.mean(hits.astype(np.float32) / np.float32(top_k)))


class GLIDE:
    """Small-path index (reference ``GLIDE<float, uint32_t>``, glide.cuh:14-189)."""

    def __init__(self, ctx: Context, graph_degree: int, data, centroids, metric: Metric = Metric.Euclidean):
        # ctor uploads data and centroids (glide_impl.cuh:15-29)
        self.ctx = ctx
        self.metric = metric
        self.d_data = self._to_device(data, torch.float32)
        self.d_centroids = self._to_device(centroids, torch.float32)
        self.d_graph = _u32_tensor(ctx, (self.d_data.shape[0], graph_degree))
        self.d_graph.fill_(-1)
        self.d_start_points = None
        self.stage_seconds: dict[str, float] = {}

    def _to_device(self, x, dtype):
        if isinstance(x, torch.Tensor):
            return x.to(self.ctx.torch_device, dtype).contiguous()
        return torch.from_numpy(np.ascontiguousarray(x)).to(self.ctx.torch_device, dtype)

    # accessors (glide.cuh:127-180)
    def num(self) -> int: return self.d_data.shape[0]
    def dim(self) -> int: return self.d_data.shape[1]
    def graph_degree(self) -> int: return self.d_graph.shape[1]
    def centroid_num(self) -> int: return self.d_centroids.shape[0]
    def start_point_num(self) -> int: return 0 if self.d_start_points is None else self.d_start_points.shape[0]
    def data_view(self) -> torch.Tensor: return self.d_data
    def graph_view(self) -> torch.Tensor: return self.d_graph
    def centroid_view(self) -> torch.Tensor: return self.d_centroids
    def start_point_view(self) -> torch.Tensor: return self.d_start_points

    def load(self, h_graph, h_start_points):
        """glide_impl.cuh:31-41."""
        g = np.ascontiguousarray(h_graph, np.uint32)
        if g.shape != tuple(self.d_graph.shape):
            raise ValueError(f"graph shape {g.shape} does not match index {tuple(self.d_graph.shape)}")
        self.d_graph = from_u32(self.ctx, g)
        self.d_start_points = from_u32(self.ctx, np.ascontiguousarray(h_start_points, np.uint32))

    def build(self, build_param: IndexParameter, search_param_knn: SearchParameter,
              search_param_refine: SearchParameter, d_knn_graph: torch.Tensor, h_segment_start, h_segment_length,
              d_map: torch.Tensor, d_reorder_data: torch.Tensor, seed: int = 0, refine_wave_rows: int | None = None):
        """``GLIDE::build`` (glide_impl.cuh:319-368): start points, subgraph build + boundary merge,
        reverse edges, refinement when search_param_refine.beam != 0. Returns kernel seconds."""
        ctx = self.ctx
        seg_start = np.ascontiguousarray(h_segment_start, np.uint32)
        seg_len = np.ascontiguousarray(h_segment_length, np.uint32)
        h_map = to_u32(d_map)
        local, original = start_point_select(seg_start, seg_len, h_map, seed)
        d_local = from_u32(ctx, local)
        times = {}
        self.d_graph.fill_(-1)
        ctx.sync_inputs()
        pk = _params_c(search_param_knn)
        ctx.check(ctx.lib.glide_subgraph_build_and_merge(
            ctx.handle, _ptr(d_reorder_data), d_reorder_data.shape[0], self.dim(), _ptr(d_knn_graph),
            d_knn_graph.shape[1], _ptr(seg_start), _ptr(seg_len), seg_start.size, _ptr(d_local), _ptr(d_map), self.num(),
            self.graph_degree(), C.byref(pk), build_param.relaxant_factor, int(self.metric), 0, _ptr(self.d_graph)))
        times["subgraph_build_and_merge"] = ctx.last_kernel_seconds
        self.d_start_points = from_u32(ctx, original)  # glide_impl.cuh:353-356
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_reverse_graph(ctx.handle, _ptr(self.d_graph), self.num(), self.graph_degree()))
        times["reverse_graph"] = ctx.last_kernel_seconds
        if search_param_refine.beam != 0:  # glide_impl.cuh:360-362
            pr = _params_c(search_param_refine)
            args = (ctx.handle, _ptr(self.d_data), self.num(), self.dim(), _ptr(self.d_graph), self.graph_degree(),
                    _ptr(self.d_centroids), self.centroid_num(), _ptr(self.d_start_points), C.byref(pr),
                    build_param.relaxant_factor, int(self.metric))
            if refine_wave_rows is None:    # the library's default wave size
                ctx.check(ctx.lib.glide_refine(*args))
            else:
                ctx.check(ctx.lib.glide_refine_waves(*args, refine_wave_rows))
            times["refine"] = ctx.last_kernel_seconds
        self.stage_seconds = times
        return sum(times.values())

    def search(self, param: SearchParameter, d_query: torch.Tensor):
        """``GLIDE::search`` (glide_impl.cuh:370-454) with device queries.
        Returns (ids uint32 [Q,k], dists float32 [Q,k]) on the host and the kernel seconds."""
        ctx = self.ctx
        q = d_query.shape[0]
        d_ids = _u32_tensor(ctx, (q, param.top_k))
        d_dists = ctx.empty((q, param.top_k), torch.float32)
        pc = _params_c(param)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_search(ctx.handle, _ptr(self.d_data), self.num(), self.dim(), _ptr(self.d_graph),
                                       self.graph_degree(), _ptr(self.d_centroids), self.centroid_num(),
                                       _ptr(self.d_start_points), _ptr(d_query), q, C.byref(pc), int(self.metric),
                                       _ptr(d_ids), _ptr(d_dists)))
        seconds = ctx.last_kernel_seconds
        return to_u32(d_ids), d_dists.cpu().numpy(), seconds

    def search_host(self, param: SearchParameter, h_query: np.ndarray, h_ids: np.ndarray | None = None,
                    h_dists: np.ndarray | None = None):
        """Host queries in, host results out: the copies are inside the call."""
        ctx = self.ctx
        h_query = np.ascontiguousarray(h_query, np.float32)
        if h_query.ndim != 2 or h_query.shape[1] != self.dim():
            raise ValueError(f"queries must be Q x {self.dim()}")
        q = h_query.shape[0]
        for name, arr, kinds in (("h_ids", h_ids, (np.uint32, np.int32)), ("h_dists", h_dists, (np.float32,))):
            if arr is not None and (arr.dtype not in kinds or arr.shape != (q, param.top_k) or not arr.flags.c_contiguous):
                raise TypeError(f"{name} must be a C-contiguous {q} x {param.top_k} array of {kinds[0].__name__}")
        if h_ids is None:
            h_ids = np.empty((q, param.top_k), np.uint32)
        if h_dists is None:
            h_dists = np.empty((q, param.top_k), np.float32)
        pc = _params_c(param)
        ctx.check(ctx.lib.glide_search_host(ctx.handle, _ptr(self.d_data), self.num(), self.dim(), _ptr(self.d_graph),
                                            self.graph_degree(), _ptr(self.d_centroids), self.centroid_num(),
                                            _ptr(self.d_start_points), _ptr(h_query), q, C.byref(pc),
                                            int(self.metric), _ptr(h_ids), _ptr(h_dists)))
        return h_ids, h_dists

    def search_pipe(self, max_queries: int, max_top_k: int, depth: int = 3) -> "SearchPipe":
        """Host-buffer search with `depth` batches in flight (`glide_search_pipe_*`)."""
        return SearchPipe(self, max_queries, max_top_k, depth)


class SearchPipe:
    """`glide_search_host` with several batches in flight: `submit` enqueues the upload, the kernels
    and the download of one batch and returns its slot, `wait(slot)` returns when the batch's
    results are in the arrays given to `submit`. Pass pinned arrays (`large.pinned_empty`), which
    must stay alive and untouched until `wait`."""

    def __init__(self, index: "GLIDE", max_queries: int, max_top_k: int, depth: int = 3):
        self.index, self.ctx = index, index.ctx
        self._h = C.c_void_p()
        self.ctx.check(self.ctx.lib.glide_search_pipe_create(self.ctx.handle, int(max_queries), index.dim(), int(max_top_k),
                                                             int(depth), C.byref(self._h)))
        self.depth = int(depth)

    def submit(self, param: SearchParameter, h_query: np.ndarray, h_ids: np.ndarray, h_dists: np.ndarray) -> int:
        ix = self.index
        q = h_query.shape[0]
        if h_query.dtype != np.float32 or h_query.ndim != 2 or h_query.shape[1] != ix.dim() or not h_query.flags.c_contiguous:
            raise TypeError(f"queries must be a C-contiguous Q x {ix.dim()} float32 array")
        for name, arr, kinds in (("h_ids", h_ids, (np.uint32, np.int32)), ("h_dists", h_dists, (np.float32,))):
            if arr.dtype not in kinds or arr.shape != (q, param.top_k) or not arr.flags.c_contiguous:
                raise TypeError(f"{name} must be a C-contiguous {q} x {param.top_k} array of {kinds[0].__name__}")
        pc = _params_c(param)
        slot = C.c_uint32()
        self.ctx.check(self.ctx.lib.glide_search_pipe_submit(
            self._h, _ptr(ix.d_data), ix.num(), ix.dim(), _ptr(ix.d_graph), ix.graph_degree(), _ptr(ix.d_centroids),
            ix.centroid_num(), _ptr(ix.d_start_points), _ptr(h_query), q, C.byref(pc), int(ix.metric), _ptr(h_ids),
            _ptr(h_dists), C.byref(slot)))
        return slot.value

    def wait(self, slot: int) -> None:
        self.ctx.check(self.ctx.lib.glide_search_pipe_wait(self._h, int(slot)))

    def drain(self) -> None:
        for s in range(self.depth):
            self.wait(s)

    def close(self) -> None:
        if self._h:
            self.ctx.lib.glide_search_pipe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
