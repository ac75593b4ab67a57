"""World-size-2 (and 3) gloo ranks on CPU: the sharded build's orchestration (kNN rows by partition
owner, build rows by reorder position, boundary rows packed and scattered, refine in waves, each
exchanged with one in-place all-gather) over the CPU oracle must give the graph and the kNN graph
the single-process oracle pipeline gives."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from glide_b200 import sharded  # noqa: E402


def test_split_range_is_a_partition():
    for n in (0, 1, 7, 100, 1001):
        for world in (1, 2, 3, 8):
            parts = [sharded.split_range(n, world, r) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1


def test_owner_ranges_cover_all_partitions_in_order():
    rng = np.random.default_rng(0)
    for world in (1, 2, 3, 8):
        for lens in ([5], [10, 10], [100, 200, 300, 50], list(rng.integers(1, 40000, 37)), [977] * 1024 + [300]):
            r = sharded.owner_ranges(lens, world)
            assert len(r) == world and r[0][0] == 0 and r[-1][1] == len(lens)
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1)) and all(a <= b for a, b in r)
    # equal partitions split evenly
    assert [b - a for a, b in sharded.owner_ranges([1000] * 64, 8)] == [8] * 8


class OracleBackend:
    """The stage calls of sharded.build_sharded over the CPU restatement of the kernels."""

    def __init__(self, base, P, graph_i32, knn_i32):
        import oracle
        self.o, self.base, self.P = oracle, base, P
        self.graph, self.knn = graph_i32, knn_i32

    def _g(self):
        return self.graph.numpy().view(np.uint32)

    def knn_segments(self, lo, hi):
        # the exact per-partition kNN rows the single-process pipeline used (a pure function of the partition)
        P = self.P
        first = int(P["seg_start"][lo])
        end = int(P["seg_start"][hi - 1]) + int(P["seg_len"][hi - 1])
        self.knn[first:end] = torch.from_numpy(P["knn"][first:end])
        return 0.0

    def build_rows(self, first, count, out):
        o, P, n = self.o, self.P, self.base.shape[0]
        if count == 0:
            return 0.0
        knn = self.knn.numpy().view(np.uint32)
        tmp = np.full((n, self.graph.shape[1]), 0xFFFFFFFF, np.uint32)
        o.build_rows(P["reorder_data"], knn, P["seg_start"], P["seg_len"], P["local_sp"], P["mapping"], n, tmp.shape[1],
                     P["p_build"], P["alpha"], P["metric"], P["order"], graph=tmp, first=first, count=count, threads=1)
        out.copy_(torch.from_numpy(tmp[P["mapping"][first:first + count]].view(np.int32)))
        return 0.0

    def build_boundary(self, first, count):
        o, P, n = self.o, self.P, self.base.shape[0]
        if count == 0:
            return 0.0
        g = self._g()
        full = g.copy()
        o.build_boundary(P["reorder_data"], self.knn.numpy().view(np.uint32), n, int(P["local_sp"][-1]), P["mapping"], full,
                         P["p_build"], P["alpha"], P["metric"], P["order"], threads=1)
        rows = P["mapping"][first:first + count]
        g[rows] = full[rows]
        return 0.0

    def reverse(self):
        self.o.reverse_graph(self._g())
        return 0.0

    def refine_rows(self, first, count, out):
        o, P = self.o, self.P
        if count == 0:
            return 0.0
        res = o.refine(self.base, self._g(), P["centroids"], P["orig_sp"], P["p_refine"], P["alpha"], P["metric"],
                       P["order"], threads=1)
        out.copy_(torch.from_numpy(res[first:first + count].view(np.int32)))
        return 0.0


WAVE = 500


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import helpers
    import oracle
    base, _ = helpers.small_dataset("int", 1200, 16, 10, seed=4)
    P = helpers.oracle_pipeline(base, centroid_num=3, boundary_factor=1.15, with_refine=False)
    want = oracle.refine(base, P["after_reverse"], P["centroids"], P["orig_sp"], P["p_refine"], P["alpha"], P["metric"],
                         P["order"], wave_rows=WAVE)
    n = base.shape[0]
    graph = torch.full((n, 16), -1, dtype=torch.int32)
    knn = torch.zeros(P["knn"].shape, dtype=torch.int32)
    backend = OracleBackend(base, P, graph, knn)
    coll = sharded.TorchCollectives(dist, world, rank)
    sharded.build_sharded(backend, coll, n, int(P["seg_len"][-1]), P["seg_start"], P["seg_len"],
                          torch.from_numpy(P["mapping"].astype(np.int64)), wave_rows=WAVE)
    ok = np.array_equal(graph.numpy().view(np.uint32), want) and np.array_equal(knn.numpy(), P["knn"])
    open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_build_equals_single_process(tmp_path, world):
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


# ---- large path: partitions owned by ranks, per-rank top-k lists gathered and merged ----
def _large_worker(rank, world, port, out_dir):
    """What bench.py's large path does with more than one rank, over the oracle: every rank searches
    the partitions it owns for all queries, the result sets are all-gathered in rank order and folded
    with the reference's merge network; the fold must give the single-process search's distances, and
    its ids wherever distances do not tie."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import golden_cases
    import oracle
    L = golden_cases.large_inputs()
    q, C, top_k = L["queries"], L["C"], 10
    Q = q.shape[0]
    o = oracle.SearchParams.derive(64, golden_cases.LARGE_DEGREE, top_k=top_k)
    routes = oracle.select_segments(q, L["centroids"], 2, 1.2)
    INVALID, FAR = 0xFFFFFFFF, np.finfo(np.float32).max

    def search(parts):
        ids, d = np.full((Q, top_k), INVALID, np.uint32), np.full((Q, top_k), FAR, np.float32)
        for s in parts:
            p = L["parts"][s]
            oracle.search_on_sub(p["rows"], p["graph"], p["map"], p["sp"], q, routes, s, o, ids, d)
        return ids, d

    lo, hi = sharded.owner_ranges(L["seg_len"][:C], world)[rank]
    mine_ids, mine_d = search(range(lo, hi))
    set_ids = torch.zeros((world * Q, top_k), dtype=torch.int32)
    set_d = torch.zeros((world * Q, top_k), dtype=torch.float32)
    set_ids[rank * Q:(rank + 1) * Q] = torch.from_numpy(mine_ids.view(np.int32))
    set_d[rank * Q:(rank + 1) * Q] = torch.from_numpy(mine_d)
    coll = sharded.TorchCollectives(dist, world, rank)
    coll.all_gather_v(set_ids, [r * Q for r in range(world)], [Q] * world)
    coll.all_gather_v(set_d, [r * Q for r in range(world)], [Q] * world)
    got_ids, got_d = oracle.merge_results(set_ids.numpy().view(np.uint32).reshape(world, Q, top_k),
                                          set_d.numpy().reshape(world, Q, top_k))
    want_ids, want_d = search(range(C))
    same_rows = (np.sort(got_ids, axis=1) == np.sort(want_ids, axis=1)).all(axis=1)
    ok = np.array_equal(got_d, want_d) and same_rows.mean() > 0.97
    open(os.path.join(out_dir, f"large{rank}.txt"), "w").write("ok" if ok else f"mismatch {same_rows.mean()}")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_large_path_owner_search_and_merge_equal_single_process(tmp_path, world):
    port = 31500 + (os.getpid() % 2000) + world
    mp.spawn(_large_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"large{r}.txt").read() == "ok"
