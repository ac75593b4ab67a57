"""Large path: the data set lives in host memory and partitions are streamed through the GPU
one at a time (reference ``GLIDE_large``, glide_large.cuh:14-212, glide_large_impl.cuh:14-507;
``preprocess_for_large`` partition.cuh:417-447; ``build_knn_for_large`` nn_descent.cuh:1515-1581).

Differences from the reference a caller will notice: rows may be fp32 or uint8 (the reference's
large path is uint8 only), every random choice is seeded, and no trailing rows are dropped (the
reference processes floor(N / batch_num) * batch_num rows, partition.cuh:231).
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


def pinned_empty(shape, dtype) -> np.ndarray:
    """Page-locked host memory as a numpy array (the array keeps its torch owner alive)."""
    t = torch.empty(shape, dtype=torch.from_numpy(np.empty(0, dtype)).dtype).pin_memory()
    a = t.numpy()
    _PINNED[id(a)] = t
    return a


_PINNED: dict = {}


def pinned_copy(a: np.ndarray) -> np.ndarray:
    out = pinned_empty(a.shape, a.dtype)
    np.copyto(out, a)
    return out


def _to_device_f32(ctx, rows: np.ndarray) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(rows)).to(ctx.torch_device)
    return t if t.dtype == torch.float32 else t.to(torch.float32)


def preprocess_for_large(ctx: api.Context, h_data: np.ndarray, centroid_num: int, sample_factor: float,
                         batch_num: int = 10, metric: Metric = Metric.Euclidean, seed: int = 0):
    """Centroids from a host-gathered sample, nearest-centroid assignment batch by batch on the GPU
    (no boundary test, partition_kernel.cuh:122-162), then the rows grouped by partition in ascending
    row order. h_data: fp32 or uint8 rows (uint8 batches cross the host link as bytes and are widened
    on the device). Returns dict(h_reorder_data (pinned, same dtype), h_map, h_segment_start,
    h_segment_length, h_centroids, seconds)."""
    n, dim = h_data.shape
    sample_num = max(centroid_num, int(n * sample_factor))
    ids = api.sample_ids(n, sample_num, seed)
    d_sample = _to_device_f32(ctx, h_data[ids])
    d_centroids, _, _ = api.kmeans_fit(ctx, d_sample, centroid_num, 0, metric, 1)
    seconds = ctx.last_kernel_seconds
    nearest = np.empty(n, np.uint32)
    batch = (n + batch_num - 1) // batch_num
    for lo in range(0, n, batch):
        hi = min(n, lo + batch)
        d_rows = _to_device_f32(ctx, h_data[lo:hi])
        d_seg, _, _ = api.define_partition(ctx, d_rows, d_centroids, -1.0, metric)
        seconds += ctx.last_kernel_seconds
        nearest[lo:hi] = api.to_u32(d_seg)[:, 0]
    reorder, order, seg_start, seg_len = _group_by_partition(h_data, nearest, centroid_num)
    return dict(h_reorder_data=reorder, h_map=order, h_segment_start=seg_start,
                h_segment_length=seg_len, h_centroids=d_centroids.cpu().numpy(), seconds=seconds)


def _group_by_partition(h_data: np.ndarray, nearest: np.ndarray, centroid_num: int):
    order = np.argsort(nearest, kind="stable").astype(np.uint32)   # ascending row id inside a partition
    seg_len = np.bincount(nearest, minlength=centroid_num).astype(np.uint32)
    seg_start = np.zeros(centroid_num, np.uint32)
    seg_start[1:] = np.cumsum(seg_len[:-1], dtype=np.uint64).astype(np.uint32)
    reorder = pinned_empty(h_data.shape, h_data.dtype)
    np.take(h_data, order, axis=0, out=reorder)
    return reorder, order, seg_start, seg_len


def matrix_file_info(ctx: api.Context, path: str, dtype) -> tuple[int, int]:
    """(rows, dim) of a matrix file (load.cuh:16-19); IOError for a missing or truncated file."""
    import ctypes as C
    rows, dim = C.c_uint32(), C.c_uint32()
    rc = ctx.lib.glide_matrix_file_info(str(path).encode(), np.dtype(dtype).itemsize, C.byref(rows), C.byref(dim))
    if rc != 0:
        raise IOError(f"{path}: missing, unreadable or shorter than its header says")
    return rows.value, dim.value


def load_rows(ctx: api.Context, path: str, dtype, first_row: int = 0, rows: int | None = None, chunk_rows: int = 0,
              threads: int = 0, d_centroids: torch.Tensor | None = None, metric: Metric = Metric.Euclidean):
    """`glide_load_rows`: rows [first_row, first_row + rows) of a matrix file into pinned memory with
    threaded positional reads; with centroids, every chunk is uploaded and assigned to its nearest
    centroid while later chunks are still being read. Returns (h_rows, h_nearest or None, stats)."""
    import ctypes as C
    dtype = np.dtype(dtype)
    if dtype not in (np.dtype(np.float32), np.dtype(np.uint8)):
        raise TypeError("matrix files hold float32 or uint8 rows")
    n, dim = matrix_file_info(ctx, path, dtype)
    rows = n - first_row if rows is None else rows
    h_rows = pinned_empty((rows, dim), dtype)
    h_nearest = pinned_empty((rows,), np.uint32) if d_centroids is not None else None
    stats = (C.c_double * 3)()
    ctx.sync_inputs()
    rc = ctx.lib.glide_load_rows(ctx.handle, str(path).encode(), dtype.itemsize, int(first_row), int(rows),
                                 h_rows.ctypes.data, int(chunk_rows), int(threads),
                                 d_centroids.data_ptr() if d_centroids is not None else None,
                                 d_centroids.shape[0] if d_centroids is not None else 0, int(metric),
                                 h_nearest.ctypes.data if h_nearest is not None else None, stats)
    if rc == -5:
        raise IOError(ctx.lib.glide_last_error(ctx.handle).decode())
    ctx.check(rc)
    return h_rows, h_nearest, dict(read_seconds=stats[0], total_seconds=stats[1], device_waited_seconds=stats[2],
                                   bytes=rows * dim * dtype.itemsize)


def preprocess_file_for_large(ctx: api.Context, path: str, dtype, centroid_num: int, sample_factor: float,
                              metric: Metric = Metric.Euclidean, seed: int = 0, chunk_rows: int = 0, threads: int = 0):
    """`preprocess_for_large` from a matrix file: the sample rows are read first (a few positional
    reads), k-means gives the centroids, then the file streams into pinned memory while the GPU
    assigns the chunks already read. Same result as `preprocess_for_large` on the loaded array."""
    dtype = np.dtype(dtype)
    n, dim = matrix_file_info(ctx, path, dtype)
    sample_num = max(centroid_num, int(n * sample_factor))
    ids = api.sample_ids(n, sample_num, seed)
    on_disk = np.memmap(path, dtype=dtype, mode="r", offset=8, shape=(n, dim))
    d_sample = _to_device_f32(ctx, np.asarray(on_disk[ids]))
    del on_disk
    d_centroids, _, _ = api.kmeans_fit(ctx, d_sample, centroid_num, 0, metric, 1)
    seconds = ctx.last_kernel_seconds
    h_rows, nearest, stats = load_rows(ctx, path, dtype, 0, n, chunk_rows, threads, d_centroids, metric)
    reorder, order, seg_start, seg_len = _group_by_partition(h_rows, nearest, centroid_num)
    return dict(h_reorder_data=reorder, h_map=order, h_segment_start=seg_start, h_segment_length=seg_len,
                h_centroids=d_centroids.cpu().numpy(), seconds=seconds, load=stats)


def _partition_list(partitions):
    """(array kept alive, pointer, count) for a partition list argument; None is the C side's null
    list, which stands for every partition in index order."""
    if partitions is None:
        return None, None, 0
    parts = np.ascontiguousarray(partitions, np.uint32)
    return parts, parts.ctypes.data, parts.size


def build_knn_for_large(ctx: api.Context, param: NNDescentParameter, h_reorder_data: np.ndarray, h_segment_start,
                        h_segment_length, metric: Metric = Metric.Euclidean, seed: int = 0,
                        exact_max_rows: int = 0xFFFFFFFF):
    """kNN graph of every partition, one resident partition at a time (build_knn_for_large,
    nn_descent.cuh:1515-1581). Returns (h_knn int32, seconds). GLIDE_large.build computes the same rows
    itself when it is not handed a kNN graph, without the round trip through host memory."""
    rows = h_reorder_data.shape[0]
    degree = min(param.graph_degree, param.intermediate_graph_degree)
    h_knn = np.zeros((rows, degree), np.int32)
    seconds = 0.0
    import ctypes as C
    for s, l in zip(h_segment_start, h_segment_length):
        s, l = int(s), int(l)
        if l == 0:
            continue
        d_part = _to_device_f32(ctx, h_reorder_data[s:s + l])
        d_knn = torch.empty((l, degree), dtype=torch.int32, device=ctx.torch_device)
        start, length = np.array([0], np.uint32), np.array([l], np.uint32)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_build_nnd_range(ctx.handle, d_part.data_ptr(), l, d_part.shape[1], start.ctypes.data,
                                                length.ctypes.data, 1, degree, param.max_iterations,
                                                param.termination_threshold, 0, exact_max_rows, seed, int(metric), s,
                                                d_knn.data_ptr(), None))
        seconds += ctx.last_kernel_seconds
        h_knn[s:s + l] = d_knn.cpu().numpy()
    return h_knn, seconds


class GLIDE_large:
    """Host-resident index over disjoint partitions (glide_large.cuh:14-212) on top of the library's
    streaming object (`glide_large_*`): rows and graph in pinned host memory, two device slots,
    uploads / kernels / downloads on three streams, partitions kept in HBM up to a budget for search."""

    def __init__(self, ctx: api.Context, graph_degree: int, metric: Metric, h_reorder_data: np.ndarray, h_map,
                 h_centroids, h_segment_start, h_segment_length, row_offset: int = 0):
        """row_offset > 0: this process holds only the reorder rows [row_offset, row_offset + len(h_reorder_data))
        (a rank of a multi-GPU run holds the rows of its own partitions); the segment tables still
        describe every partition, and only partitions inside that range may be built or searched here."""
        import ctypes as C
        self.ctx, self.metric = ctx, metric
        if h_reorder_data.dtype not in (np.float32, np.uint8):
            raise TypeError("rows must be float32 or uint8")
        self.h_data = h_reorder_data if (id(h_reorder_data) in _PINNED and h_reorder_data.flags.c_contiguous) \
            else pinned_copy(np.ascontiguousarray(h_reorder_data))
        self.h_map = np.ascontiguousarray(h_map, np.uint32)
        self.h_centroids = np.ascontiguousarray(h_centroids, np.float32)
        self.seg_start = np.ascontiguousarray(h_segment_start, np.uint32)
        self.seg_len = np.ascontiguousarray(h_segment_length, np.uint32)
        self.row_offset = int(row_offset)
        if self.h_map.shape[0] != self.h_data.shape[0]:
            raise ValueError("one map entry per held row expected")
        self.h_graph = pinned_empty((self.h_data.shape[0], graph_degree), np.uint32)
        self.h_graph.fill(api.INVALID)
        self.stage_seconds: dict[str, float] = {}
        self.stats: dict = {}
        self.d_centroids = torch.from_numpy(self.h_centroids).to(ctx.torch_device)
        handle = C.c_void_p()
        off = self.row_offset   # the library indexes by global reorder row: hand it where row 0 would lie
        ctx.check(ctx.lib.glide_large_create(
            ctx.handle, self.h_data.ctypes.data - off * self.h_data.shape[1] * self.h_data.itemsize,
            1 if self.h_data.dtype == np.uint8 else 0, self.h_data.shape[1], self.seg_start.ctypes.data,
            self.seg_len.ctypes.data, self.seg_start.size, self.h_map.ctypes.data - off * 4, graph_degree, int(metric),
            self.h_graph.ctypes.data - off * graph_degree * 4, C.byref(handle)))
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None):
            self.ctx.lib.glide_large_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def num(self): return self.h_data.shape[0]
    def dim(self): return self.h_data.shape[1]
    def graph_degree(self): return self.h_graph.shape[1]
    def segment_num(self): return self.seg_start.size
    def centroids_num(self): return self.h_centroids.shape[0]
    def graph_view(self): return self.h_graph

    def start_point_view(self):
        out = np.zeros(self.segment_num(), np.uint32)
        self.ctx.check(self.ctx.lib.glide_large_get_start_points(self.handle, out.ctypes.data))
        return out

    def set_start_points(self, h_start_points) -> None:
        sp = np.ascontiguousarray(h_start_points, np.uint32)
        self.ctx.check(self.ctx.lib.glide_large_set_start_points(self.handle, sp.ctypes.data))

    def load(self, h_graph, h_start_points):
        np.copyto(self.h_graph, np.ascontiguousarray(h_graph, np.uint32))
        sp = np.ascontiguousarray(h_start_points, np.uint32)
        self.ctx.check(self.ctx.lib.glide_large_set_start_points(self.handle, sp.ctypes.data))

    def _stats(self):
        import ctypes as C
        out = (C.c_double * 8)()
        self.ctx.lib.glide_large_last_stats(self.handle, out)
        return list(out)

    def build(self, build_param: IndexParameter, search_param_knn: SearchParameter,
              search_param_refine: SearchParameter, h_knn_graph: np.ndarray | None = None, seed: int = 0,
              partitions=None, nnd: NNDescentParameter | None = None, exact_max_rows: int = 0xFFFFFFFF,
              want_knn: bool = False):
        """GLIDE_large::build (glide_large_impl.cuh:79-328) for `partitions` (default: all). Without
        h_knn_graph the kNN rows are computed on the device per partition (NN-descent or the exact
        all-pairs kernel) as part of the same streamed pass. Returns kernel seconds."""
        import ctypes as C
        ctx = self.ctx
        parts, parts_ptr, parts_n = _partition_list(partitions)
        nnd = nnd or NNDescentParameter(build_param.knn_degree)
        knn_degree = build_param.knn_degree if h_knn_graph is None else h_knn_graph.shape[1]
        pk = api._params_c(search_param_knn)
        pr = api._params_c(search_param_refine)
        knn_in = None
        if h_knn_graph is not None:
            knn_in = np.ascontiguousarray(h_knn_graph, np.int32)
        self.h_knn = pinned_empty((self.num(), knn_degree), np.int32) if want_knn else None
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_large_build(self.handle, parts_ptr, parts_n, knn_degree, C.byref(pk), C.byref(pr),
                                            build_param.relaxant_factor, nnd.max_iterations, nnd.termination_threshold, 0,
                                            exact_max_rows, seed,
                                            None if knn_in is None else knn_in.ctypes.data - self.row_offset * knn_degree * 4,
                                            None if self.h_knn is None else self.h_knn.ctypes.data - self.row_offset * knn_degree * 4))
        st = self._stats()
        self.stage_seconds = dict(knn=st[0], subgraph_build=st[1], reverse_graph=st[2], refine=st[3])
        self.stats = dict(h2d_bytes=st[4], h2d_seconds=st[5], partitions_uploaded=int(st[6]))
        return sum(self.stage_seconds.values())

    def make_resident(self, budget_bytes: int, partitions=None) -> int:
        """Keep partitions in device memory for the searches that follow; returns how many fit."""
        import ctypes as C
        parts, parts_ptr, parts_n = _partition_list(partitions)
        n = C.c_uint32(0)
        self.ctx.check(self.ctx.lib.glide_large_make_resident(self.handle, parts_ptr, parts_n, int(budget_bytes),
                                                              C.byref(n)))
        return int(n.value)

    def resident_buffers(self, partition: int):
        """Device addresses (rows fp32, graph rows, id map) of a partition's resident buffers, allocated
        uninitialised when the partition is not resident yet; see `glide_large_resident_buffers`."""
        import ctypes as C
        r, g, m = C.c_void_p(), C.c_void_p(), C.c_void_p()
        self.ctx.check(self.ctx.lib.glide_large_resident_buffers(self.handle, int(partition), C.byref(r), C.byref(g), C.byref(m)))
        return r.value or 0, g.value or 0, m.value or 0

    def replicate_partitions(self, owner_of_partition, rank: int) -> int:
        """Every rank ends up with every partition in device memory: the owner's resident buffers are
        broadcast over the context's NCCL communicator into buffers allocated here on the other ranks
        (rows as fp32, graph rows, id map). Own partitions must be resident. Returns the bytes received."""
        ctx = self.ctx
        dim, deg = self.h_data.shape[1], self.graph_degree()
        received = 0
        for p, owner in enumerate(owner_of_partition):
            ln = int(self.seg_len[p])
            if ln == 0:
                continue
            rows, graph, idmap = self.resident_buffers(p)
            for ptr, nbytes in ((rows, ln * dim * 4), (graph, ln * deg * 4), (idmap, ln * 4)):
                ctx.check(ctx.lib.glide_comm_broadcast(ctx.handle, ptr, nbytes, int(owner)))
                if owner != rank:
                    received += nbytes
        ctx.check(ctx.lib.glide_ctx_synchronize(ctx.handle))
        return received

    def search_device(self, param: SearchParameter, min_segment_num: int, boundary_factor: float, d_query: torch.Tensor,
                      partitions=None):
        """Results stay on the device: (ids int32 tensor [Q,k] of original ids, dists [Q,k], kernel seconds)."""
        import ctypes as C
        ctx = self.ctx
        q = d_query.shape[0]
        parts, parts_ptr, parts_n = _partition_list(partitions)
        d_ids = api._u32_tensor(ctx, (q, param.top_k))
        d_d = ctx.empty((q, param.top_k), torch.float32)
        pc = api._params_c(param)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_large_search(self.handle, d_query.data_ptr(), q, self.d_centroids.data_ptr(),
                                             self.centroids_num(), min_segment_num, boundary_factor, C.byref(pc),
                                             parts_ptr, parts_n, d_ids.data_ptr(), d_d.data_ptr()))
        st = self._stats()
        self.stats = dict(route_seconds=st[0], search_seconds=st[1], h2d_bytes=st[4], h2d_seconds=st[5],
                          partitions_uploaded=int(st[6]), partitions_searched=int(st[7]))
        return d_ids, d_d, st[0] + st[1]

    def build_with_merge(self, boundary_factor: float, link_count: int = 8, link_beam: int = 32):
        """The merged index (declared in the reference, glide_large.cuh:96, and defined nowhere: this
        library's own design, see `glide_large_merge`): one graph over reorder ids with links across
        partition borders, searched with one beam search per query. Every partition must be resident
        (`make_resident`). Returns dict(link_seconds, reverse_seconds, rows_with_links)."""
        import ctypes as C
        p_link = SearchParameter(top_k=link_count, beam=link_beam).derive(self.graph_degree())
        pc = api._params_c(p_link)
        stats = (C.c_double * 3)()
        self.ctx.sync_inputs()
        self.ctx.check(self.ctx.lib.glide_large_merge(self.handle, self.d_centroids.data_ptr(), self.centroids_num(),
                                                      float(boundary_factor), int(link_count), C.byref(pc), stats))
        return dict(link_seconds=stats[0], reverse_seconds=stats[1], rows_with_links=int(stats[2]))

    def merged_graph(self) -> np.ndarray:
        """The merged graph in reorder ids (rows x graph_degree)."""
        g = np.empty((self.h_data.shape[0], self.graph_degree()), np.uint32)
        self.ctx.check(self.ctx.lib.glide_large_merged_graph(self.handle, g.ctypes.data))
        return g

    def search_merged_device(self, param: SearchParameter, d_query: torch.Tensor):
        """One beam search per query over the merged graph; (ids tensor of original ids, dists, kernel seconds)."""
        import ctypes as C
        ctx = self.ctx
        q = d_query.shape[0]
        d_ids = api._u32_tensor(ctx, (q, param.top_k))
        d_d = ctx.empty((q, param.top_k), torch.float32)
        pc = api._params_c(param)
        ctx.sync_inputs()
        ctx.check(ctx.lib.glide_large_search_merged(self.handle, d_query.data_ptr(), q, self.d_centroids.data_ptr(),
                                                    self.centroids_num(), C.byref(pc), d_ids.data_ptr(), d_d.data_ptr()))
        return d_ids, d_d, ctx.last_kernel_seconds

    def search_merged(self, param: SearchParameter, d_query: torch.Tensor):
        d_ids, d_d, seconds = self.search_merged_device(param, d_query)
        return api.to_u32(d_ids), d_d.cpu().numpy(), seconds

    def search(self, param: SearchParameter, min_segment_num: int, boundary_factor: float, d_query: torch.Tensor,
               partitions=None):
        """glide_large_impl.cuh:355-507. Returns (ids uint32 [Q,k] original ids, dists [Q,k], kernel seconds)."""
        d_ids, d_d, seconds = self.search_device(param, min_segment_num, boundary_factor, d_query, partitions)
        return api.to_u32(d_ids), d_d.cpu().numpy(), seconds
