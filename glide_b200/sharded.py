"""Small-path index build sharded over the ranks of one node.

Every rank holds the data set and runs the cheap stages itself (partitioning, kNN graph,
reverse edges: together under 10 % of the build); the two expensive per-point stages are
split by contiguous row ranges and their rows exchanged:

* subgraph build (`build_kernel`): rank r builds reorder rows split(num, world, r); rows are
  keyed by ORIGINAL id, each written by exactly one rank into a graph that starts as all
  0xffffffff (-1 as int32), so one all-reduce(MAX) over the int32 view merges them;
* boundary build (`build_boundary_kernel`): rank r handles its share of the boundary copies;
  the rows they merged into (`map[copy]`, known to every rank) are broadcast from their owner;
* refine: rank r refines points split(num, world, r) against a snapshot every rank shares and
  broadcasts its contiguous rows.

The result is identical to the single-GPU build. The stage implementations come from a
backend object so that the orchestration can be tested with CPU ranks (gloo) over the oracle.
"""
from __future__ import annotations

import numpy as np
import torch


def split_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced: the first n % world ranks get one extra row."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class Collectives:
    """The three exchanges the build needs, over torch.distributed (NCCL on GPUs, gloo on CPU)."""

    def __init__(self, dist=None, world: int = 1, rank: int = 0):
        self.dist, self.world, self.rank = dist, world, rank

    def merge_disjoint_rows(self, graph_i32: torch.Tensor):
        """Rows written by exactly one rank over a -1-filled graph."""
        if self.world > 1:
            self.dist.all_reduce(graph_i32, op=self.dist.ReduceOp.MAX)

    def exchange_rows(self, graph_i32: torch.Tensor, row_ids_per_rank: list[torch.Tensor]):
        """row_ids_per_rank[r]: the rows rank r has updated (known to every rank)."""
        if self.world == 1:
            return
        for r, idx in enumerate(row_ids_per_rank):
            if idx.numel() == 0:
                continue
            buf = graph_i32[idx].contiguous() if r == self.rank else torch.empty(
                (idx.numel(), graph_i32.shape[1]), dtype=graph_i32.dtype, device=graph_i32.device)
            self.dist.broadcast(buf, src=r)
            if r != self.rank:
                graph_i32[idx] = buf

    def exchange_ranges(self, graph_i32: torch.Tensor, n: int):
        if self.world == 1:
            return
        for r in range(self.world):
            lo, hi = split_range(n, self.world, r)
            if hi > lo:
                self.dist.broadcast(graph_i32[lo:hi], src=r)


def build_sharded(backend, coll: Collectives, num: int, boundary_num: int, graph_i32: torch.Tensor,
                  map_ids: torch.Tensor, do_refine: bool = True) -> dict:
    """graph_i32: num x degree, all -1 on entry, the finished graph on return (on every rank).
    map_ids: reorder id -> original id (long tensor on the graph's device).
    backend: build_range(first_row, row_count), reverse(), refine_range(snapshot, first, count);
    each returns its kernel seconds and works on graph_i32 in place."""
    seconds = {}
    lo, hi = split_range(num, coll.world, coll.rank)
    seconds["subgraph_build"] = backend.build_range(lo, hi - lo)
    coll.merge_disjoint_rows(graph_i32)
    if boundary_num > 0:
        blo, bhi = split_range(boundary_num, coll.world, coll.rank)
        seconds["boundary_build"] = backend.build_range(num + blo, bhi - blo)
        rows = []
        for r in range(coll.world):
            a, b = split_range(boundary_num, coll.world, r)
            rows.append(map_ids[num + a:num + b])
        coll.exchange_rows(graph_i32, rows)
    seconds["reverse_graph"] = backend.reverse()
    if do_refine:
        snapshot = graph_i32.clone()
        seconds["refine"] = backend.refine_range(snapshot, lo, hi - lo)
        coll.exchange_ranges(graph_i32, num)
    return seconds
