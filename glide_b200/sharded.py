"""Small-path index build sharded over the ranks of one node (one process per GPU).

Every rank holds the data set (the small path is the GPU-resident one) and runs the cheap,
order-sensitive stages itself: centroids, assignment, slots, reorder, reverse edges. The three
expensive stages are split, and what crosses NVLink is rows of ids, never vectors:

* kNN graph: partitions are the unit. Consecutive partitions (the boundary partition is the last
  one) go to consecutive ranks, balanced by estimated cost; a rank builds the kNN rows of its own
  partitions and one in-place all-gather of those rows gives every rank the whole kNN graph.
* subgraph build (`build_kernel`): rank r builds an equal share of the reorder rows and writes
  them BY REORDER POSITION, so its rows are one contiguous block; one all-gather, then every rank
  scatters the rows to their original ids through the map. Boundary copies
  (`build_boundary_kernel`) are split evenly too; the rows they merge into are packed in boundary
  order, gathered, and scattered back.
* refine: waves of consecutive ids (as on one GPU); every wave is split evenly over the ranks,
  its rows gathered, then written back before the next wave starts.

Each exchange is one `all_gather_v` (rank r owns a contiguous block of rows of a buffer every rank
holds). The result equals the single-GPU build bit for bit. Stage implementations come from a
backend object and the exchange from a collectives object, so the orchestration also runs on CPU
ranks (gloo) over the CPU restatement of the kernels, which is how it is tested without GPUs.
"""
from __future__ import annotations

import numpy as np
import torch


def split_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced: the first n % world ranks get one extra row."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def split_all(n: int, world: int) -> tuple[list[int], list[int]]:
    """Offsets and counts of split_range for every rank."""
    parts = [split_range(n, world, r) for r in range(world)]
    return [a for a, _ in parts], [b - a for a, b in parts]


def knn_cost(length: int, exact_max_rows: int = 16384) -> float:
    """Relative cost of one partition's kNN graph: all pairs up to exact_max_rows rows, NN-descent
    (a few thousand distance evaluations per row) beyond."""
    return float(length) * float(min(length, exact_max_rows)) if length <= exact_max_rows else float(length) * 6000.0


def owner_ranges(seg_len, world: int, exact_max_rows: int = 16384) -> list[tuple[int, int]]:
    """Consecutive partitions to consecutive ranks, balanced by knn_cost: rank r owns segments
    [lo_r, hi_r) (possibly none when there are fewer partitions than ranks). The cut before rank r is
    the partition boundary whose cost prefix lies nearest to r/world of the total."""
    costs = np.array([knn_cost(int(l), exact_max_rows) for l in seg_len], np.float64)
    S = costs.size
    before = np.concatenate([[0.0], np.cumsum(costs)])   # before[s] = cost of partitions 0 .. s-1
    cuts = [0]
    for r in range(1, world):
        target = before[-1] * r / world
        s = int(np.searchsorted(before, target, side="left"))   # before[s-1] < target <= before[s]
        s = min(max(s, 1), S)
        cut = s - 1 if target - before[s - 1] <= before[s] - target else s
        cuts.append(min(max(cut, cuts[-1]), S))
    cuts.append(S)
    return [(cuts[r], cuts[r + 1]) for r in range(world)]


class Collectives:
    """The one exchange the build needs. This base class is the single-rank case."""
    world, rank = 1, 0

    def all_gather_v(self, rows: torch.Tensor, offsets: list[int], counts: list[int]) -> None:
        """In place: rank r owns rows [offsets[r], offsets[r] + counts[r]) of the 2-D contiguous tensor
        `rows`; afterwards every rank holds every block."""

    def sync(self) -> None:
        """Wait until the exchanges issued so far are done (before the host or another stream reads them)."""


class TorchCollectives(Collectives):
    """Over torch.distributed (gloo ranks on CPU in the tests)."""

    def __init__(self, dist, world: int, rank: int):
        self.dist, self.world, self.rank = dist, world, rank

    def all_gather_v(self, rows, offsets, counts):
        if self.world == 1:
            return
        for r in range(self.world):
            if counts[r]:
                self.dist.broadcast(rows[offsets[r]:offsets[r] + counts[r]], src=r)


class GlideCollectives(Collectives):
    """NCCL through the library's own communicator (`glide_comm_*`): the collective is enqueued on the
    context's stream, in order with the kernels that produce the rows."""

    def __init__(self, ctx):
        self.ctx = ctx
        self.world = int(ctx.lib.glide_comm_world(ctx.handle))
        self.rank = int(ctx.lib.glide_comm_rank(ctx.handle))

    def all_gather_v(self, rows, offsets, counts):
        if self.world == 1:
            return
        assert rows.is_contiguous() and rows.dim() == 2
        row_bytes = rows.shape[1] * rows.element_size()
        off = np.asarray(offsets, np.uint64) * np.uint64(row_bytes)
        cnt = np.asarray(counts, np.uint64) * np.uint64(row_bytes)
        self.ctx.sync_inputs()   # what torch wrote into `rows` is visible to the context's stream
        self.ctx.check(self.ctx.lib.glide_comm_all_gather_v(self.ctx.handle, rows.data_ptr(), off.ctypes.data, cnt.ctypes.data))

    def sync(self):
        if self.world > 1:
            self.ctx.check(self.ctx.lib.glide_ctx_synchronize(self.ctx.handle))


def build_sharded(backend, coll: Collectives, num: int, boundary_num: int, seg_start, seg_len, map_ids: torch.Tensor,
                  do_refine: bool = True, wave_rows: int = 65536, exact_max_rows: int = 16384) -> dict:
    """backend (all buffers live on the backend's device, every rank holds all of them):
      knn          (num + boundary_num) x knn_degree int32
      graph        num x degree int32, all -1 on entry, the finished graph on return
      knn_segments(lo, hi)                 kNN rows of partitions [lo, hi) into knn
      build_rows(first, count, out)        build_kernel rows of reorder ids [first, first+count) into out (count x degree)
      build_boundary(first, count)         build_boundary_kernel for reorder ids [first, first+count), editing graph
      reverse()                            reverse edges on graph
      refine_rows(first, count, out)       refined rows of points [first, first+count) read from graph, into out
    each returning its kernel seconds. seg_start/seg_len: C + 1 entries, the last the boundary partition.
    map_ids: reorder id -> original id (long tensor on the device)."""
    world, rank = coll.world, coll.rank
    seconds = {}
    graph, knn = backend.graph, backend.knn
    degree = graph.shape[1]
    dev = graph.device

    # ---- kNN graph by partition owner ----
    owners = owner_ranges(seg_len, world, exact_max_rows)
    lo, hi = owners[rank]
    seconds["knn"] = backend.knn_segments(lo, hi) if hi > lo else 0.0
    ends = [int(seg_start[h - 1]) + int(seg_len[h - 1]) if h > l else None for l, h in owners]
    offsets = [int(seg_start[l]) if h > l else 0 for l, h in owners]
    counts = [(e - o) if e is not None else 0 for e, o in zip(ends, offsets)]
    coll.all_gather_v(knn, offsets, counts)
    coll.sync()

    # ---- subgraph build, rows by reorder position ----
    rows_rr = torch.empty((num, degree), dtype=graph.dtype, device=dev)
    offs, cnts = split_all(num, world)
    seconds["subgraph_build"] = backend.build_rows(offs[rank], cnts[rank], rows_rr[offs[rank]:offs[rank] + cnts[rank]])
    coll.all_gather_v(rows_rr, offs, cnts)
    coll.sync()
    graph[map_ids[:num]] = rows_rr            # map[:num] is a permutation of the original ids
    del rows_rr

    # ---- boundary copies ----
    if boundary_num > 0:
        boffs, bcnts = split_all(boundary_num, world)
        b0, bc = boffs[rank], bcnts[rank]
        seconds["boundary_build"] = backend.build_boundary(num + b0, bc)
        packed = torch.empty((boundary_num, degree), dtype=graph.dtype, device=dev)
        packed[b0:b0 + bc] = graph[map_ids[num + b0:num + b0 + bc]]
        coll.all_gather_v(packed, boffs, bcnts)
        coll.sync()
        graph[map_ids[num:num + boundary_num]] = packed   # a point has at most one boundary copy: no row is written twice
        del packed

    seconds["reverse_graph"] = backend.reverse()

    # ---- refine in waves ----
    if do_refine:
        if wave_rows <= 0 or wave_rows > num:
            wave_rows = num
        wave = torch.empty((wave_rows, degree), dtype=graph.dtype, device=dev)
        total = 0.0
        for wlo in range(0, num, wave_rows):
            wn = min(wave_rows, num - wlo)
            woffs, wcnts = split_all(wn, world)
            total += backend.refine_rows(wlo + woffs[rank], wcnts[rank], wave[woffs[rank]:woffs[rank] + wcnts[rank]])
            coll.all_gather_v(wave, woffs, wcnts)
            coll.sync()
            graph[wlo:wlo + wn] = wave[:wn]
        seconds["refine"] = total
    return seconds
